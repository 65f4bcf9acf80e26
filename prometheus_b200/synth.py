"""Synthetic data generation: the Python face of ``native.synth``.

Re-exports the C++ implementation (style rewrites with a source-grounded fact check, rejection
sampling against verifiers, procedural ARC families with dihedral x colour augmentation,
agentic trajectories; reference ``synth/__init__.py`` :161-1331 and the ``synth`` crate) and adds
the two adapters that connect it to the rest of this package: a generator backed by the batch
generation engine and a grid tokenizer backed by ``tokenizer.Tokenizer.encode_grid``.
``synth_twin`` states the same rules a second time in Python / NumPy; the two are checked
against each other on generated inputs.
"""
from __future__ import annotations

from .native import serve as _serve
from .native import synth as _s

SCHEMA_VERSION = _s.SCHEMA_VERSION
DEFAULT_MAX_TOKENS, DEFAULT_TEMPERATURE, DEFAULT_MAX_BATCH = _s.DEFAULT_MAX_TOKENS, _s.DEFAULT_TEMPERATURE, _s.DEFAULT_MAX_BATCH
DEFAULT_N_SAMPLES = _s.DEFAULT_N_SAMPLES
STYLES, DOMAINS = tuple(_s.STYLES), tuple(_s.DOMAINS)

generate_prompt, extract_claims, check_claim, fact_check, accept = (
    _s.generate_prompt, _s.extract_claims, _s.check_claim, _s.fact_check, _s.accept)
token_count, precision = _s.token_count, _s.precision
Orchestrator, RejectionSampler, Problem = _s.Orchestrator, _s.RejectionSampler, _s.Problem
generate_solve_prompt, extract_answer, verified_correct_rate = (
    _s.generate_solve_prompt, _s.extract_answer, _s.verified_correct_rate)
arc, agentic = _s.arc, _s.agentic


def engine_generator(engine: "_serve.LocalEngine"):
    """``generate(prompts, max_tokens, temperature) -> [text]`` on a ``serve.LocalEngine`` (or a
    ``serve.Router``), splitting batches at the engine's limit."""
    limit = getattr(engine, "max_batch", None) or getattr(getattr(engine, "engine", None), "max_batch", 8)

    def generate(prompts, max_tokens, temperature):
        out = []
        for i in range(0, len(prompts), limit):
            out += [c[1] for c in engine.generate(list(prompts[i:i + limit]), int(max_tokens), float(temperature))]
        return out

    return generate


def grid_tokens(tokenizer, grid) -> list:
    """Token ids of a grid: one token per cell, row-major (``tokenizer.encode_grid``)."""
    return arc.tokenize_grid(lambda cells: tokenizer.encode_grid(list(cells)), grid)
