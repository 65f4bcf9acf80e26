"""Behaviour lists of the think-span layout, the thought-segment decoder and the hidden-state
alignment (``prometheus_b200.latent``; reference tests/test_latent_segment.py, model/latent.py)
and of the seed genome loader (``prometheus_b200.genome_seed``; reference
tests/test_genome_seed.py, harness/genome-seed/genome_seed.py:16-131)."""
import dataclasses
import math
import shutil

import numpy as np
import pytest
import torch

from prometheus_b200 import genome_seed as G
from prometheus_b200 import latent as L

CFG = L.LatentConfig()
K = L.SpanKind


# ------------------------------------------------------------------------------ think layout
def test_layout_is_chunks_separated_by_one_anchor():
    plan = L.plan_think_layout([4, 8], [7, 9], CFG)
    assert plan == (L.ThinkSpan(K.LATENT, 4, ()), L.ThinkSpan(K.ANCHOR, 0, (7, 9)), L.ThinkSpan(K.LATENT, 8, ()))
    assert [s.kind for s in L.plan_think_layout([4, 4, 4], [1], CFG)] == [K.LATENT, K.ANCHOR, K.LATENT, K.ANCHOR, K.LATENT]
    assert L.plan_think_layout([64], [0], CFG) == (L.ThinkSpan(K.LATENT, 64, ()),)
    cases = [([], [1], "chunk_lengths"), ([3], [1], "chunk length"), ([65], [1], "chunk length"), ([4.0], [1], "chunk length"), ([True], [1], "chunk length"),
             ([4], [], "anchor empty"), ([4], [-1], "anchor token"), ([4], [1.0], "anchor token")]
    for lengths, anchors, text in cases:
        with pytest.raises(L.LatentError, match=text):
            L.plan_think_layout(lengths, anchors, CFG)
    with pytest.raises(L.LatentError, match="chunk_lengths"):
        L.plan_think_layout([], [], CFG)                                                 # lengths are checked before anchors
    with pytest.raises(L.LatentError, match="chunk length"):
        L.plan_think_layout([2], [], CFG)


def test_tool_spans_go_between_an_anchor_and_the_next_chunk():
    plan = L.plan_think_layout([4, 4, 4], [1], CFG)
    one = L.insert_discrete_tool(plan, 0, [50, 51])
    assert [s.kind for s in one] == [K.LATENT, K.ANCHOR, K.TOOL, K.LATENT, K.ANCHOR, K.LATENT] and one[2].token_ids == (50, 51)
    last = L.insert_discrete_tool(plan, 2, [9])
    assert [s.kind for s in last][-2:] == [K.LATENT, K.TOOL]                              # after the last chunk: appended
    two = L.insert_discrete_tool(L.insert_discrete_tool(plan, 0, [1]), 0, [2])
    assert [s.token_ids for s in two if s.kind is K.TOOL] == [(1,), (2,)]                 # repeated inserts keep their order
    twice_last = L.insert_discrete_tool(last, 2, [8])
    assert [s.token_ids for s in twice_last[-2:]] == [(9,), (8,)]
    bad_layouts = [(), "latent", None, (L.ThinkSpan(K.ANCHOR, 0, (1,)),) + plan, plan[:1] + plan[2:], plan[:2] + (plan[1],) + plan[2:],
                   (plan[0], L.ThinkSpan(K.TOOL, 0, (1,)), plan[1], plan[2]), plan + (plan[1],), (plan[0], "span")]
    for layout in bad_layouts:
        with pytest.raises(L.LatentError, match="layout"):
            L.insert_discrete_tool(layout, 0, [1])
    for after in (-1, 3, 1.0, True):
        with pytest.raises(L.LatentError, match="after_chunk"):
            L.insert_discrete_tool(plan, after, [1])
    with pytest.raises(L.LatentError, match="tool empty"):
        L.insert_discrete_tool(plan, 0, [])
    for ids in ([-1], [1.5], [True]):
        with pytest.raises(L.LatentError, match="tool token"):
            L.insert_discrete_tool(plan, 0, ids)
    with pytest.raises(L.LatentError, match="layout"):
        L.insert_discrete_tool((), 9, [])                                                 # the layout is checked first


# ------------------------------------------------------------------------------ segment decoder
def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def test_one_token_segments_use_the_tied_head_and_ignore_the_decoder():
    h, u = rnd(6, seed=1), rnd(11, 6, seed=2)
    got = L.decode_thought_segment(h, 1, u)
    torch.testing.assert_close(got, h @ u.T)
    assert torch.equal(L.decode_thought_segment(h, 1, u, decoder="not even a decoder"), got)
    w = rnd(6, seed=3).abs()
    normed = L.decode_thought_segment(h, 1, u, final_norm=w)
    torch.testing.assert_close(normed, (h * torch.rsqrt((h * h).mean() + 1e-6) * w) @ u.T)


def test_longer_segments_run_a_small_recurrent_decoder():
    h, u = rnd(5, seed=4), rnd(9, 5, seed=5)
    dec = L.SegmentDecoder(rnd(5, 5, seed=6) * 0.4, rnd(5, 5, seed=7) * 0.4, rnd(5, seed=8) * 0.1)
    got = L.decode_thought_segment(h, 3, u, dec)
    state, rows = np.zeros(5), []
    for _ in range(3):
        state = np.tanh(h.numpy() @ dec.w_in.numpy() + state @ dec.w_h.numpy() + dec.bias.numpy())
        rows.append(state @ u.numpy().T)
    np.testing.assert_allclose(got.numpy(), np.stack(rows), rtol=1e-10)
    assert got.shape == (3, 9)
    hh = h.clone().requires_grad_(True)
    w_in = dec.w_in.clone().requires_grad_(True)
    L.decode_thought_segment(hh, 2, u, L.SegmentDecoder(w_in, dec.w_h, dec.bias)).sum().backward()
    assert float(hh.grad.abs().max()) > 0 and float(w_in.grad.abs().max()) > 0


def test_decoder_argument_errors_come_in_a_fixed_order():
    h, u = rnd(4, seed=9), rnd(7, 4, seed=10)
    dec = L.SegmentDecoder(rnd(4, 4), rnd(4, 4), rnd(4))
    cases = [((h, 0, u, dec), "teacher_len"), ((h, True, u, dec), "teacher_len"), ((h, 1.0, u, dec), "teacher_len"),
             ((rnd(2, 4), 1, u, dec), "hidden"), ((torch.zeros(0, dtype=torch.float64), 1, u, dec), "hidden"),
             ((torch.tensor([math.nan] * 4), 1, u, dec), "hidden"), ((h, 1, rnd(7, 5), dec), "unembed"), ((h, 1, rnd(7), dec), "unembed"),
             ((h, 2, u, None), "decoder"), ((h, 2, u, L.SegmentDecoder(rnd(4, 3), rnd(4, 4), rnd(4))), "decoder"),
             ((h, 2, u, L.SegmentDecoder(rnd(4, 4), rnd(4, 4), torch.full((4,), math.inf, dtype=torch.float64))), "decoder")]
    for args, text in cases:
        with pytest.raises(L.LatentError, match=text):
            L.decode_thought_segment(*args)
    with pytest.raises(L.LatentError, match="teacher_len"):
        L.decode_thought_segment(rnd(2, 4), 0, rnd(7), None)                              # the length is checked first of all
    with pytest.raises(L.LatentError, match="final_norm"):
        L.decode_thought_segment(h, 1, u, final_norm=rnd(5))


# ------------------------------------------------------------------------------ alignment / objective
def test_alignment_is_a_mean_square_to_a_detached_teacher():
    s, t = rnd(3, 4, seed=11).requires_grad_(True), rnd(3, 4, seed=12).requires_grad_(True)
    loss = L.codi_alignment(s, t)
    assert float(loss) == pytest.approx(float(((s - t) ** 2).mean()))
    loss.backward()
    torch.testing.assert_close(s.grad, 2 * (s - t).detach() / 12)
    assert t.grad is None                                                                 # nothing flows into the teacher
    for a, b, text in ((rnd(4), rnd(4), "student_h"), (rnd(3, 4), rnd(4), "teacher_h"), (rnd(3, 4), rnd(3, 5), "shape"),
                       (torch.full((2, 2), math.nan, dtype=torch.float64), rnd(2, 2), "student_h"), (torch.zeros(0, 4), torch.zeros(0, 4), "student_h")):
        with pytest.raises(L.LatentError, match=text):
            L.codi_alignment(a, b)


def test_stage_b_objective_adds_the_weighted_alignment():
    halt, ans, th = rnd(3, seed=13), rnd(3, 5, seed=14), rnd(2, 5, seed=15)
    s, t = rnd(2, 4, seed=16), rnd(2, 4, seed=17)
    base = L.stage_b_loss(halt, ans, th, [1, 2], [1, 1], 3, 1, CFG)
    for w in (0.0, 1.0, 2.5):
        obj = L.stage_b_objective(halt, ans, th, [1, 2], [1, 1], 3, 1, CFG, s, t, align_weight=w)
        assert float(obj.total) == pytest.approx(float(base.total) + w * float(L.codi_alignment(s, t)))
        assert float(obj.stage_b.total) == pytest.approx(float(base.total)) and float(obj.l_align) == pytest.approx(float(L.codi_alignment(s, t)))
    for bad in (-1.0, math.nan, math.inf, True, "1"):
        with pytest.raises(L.LatentError, match="align_weight"):
            L.stage_b_objective(halt, ans, th, [1, 2], [1, 1], 3, 1, dataclasses.replace(CFG, max_thoughts=-1), s, t, align_weight=bad)   # checked first


# ------------------------------------------------------------------------------ seed genome
def test_the_shipped_seed():
    assert G.ROLES == ("director", "researcher", "implementer", "reviewer", "tester") and issubclass(G.GenomeError, ValueError)
    root = G.seed_root()
    assert root.is_dir() and all((root / d).is_dir() for d in ("roles", "programs", "tools", "skills"))
    seed = G.load_seed()
    assert G.role_names(seed) == G.ROLES and seed.root == root.resolve() and all(r.body.strip() for r in seed.roles)
    assert "loop" in [p.name for p in seed.programs]
    assert isinstance(seed.tools, tuple) and isinstance(seed.skills, tuple)
    G.require_roles(seed)
    with pytest.raises(dataclasses.FrozenInstanceError):
        seed.roles = ()
    with pytest.raises(dataclasses.FrozenInstanceError):
        seed.roles[0].body = ""
    text = G.instructions_for(seed, "reviewer")
    assert text.startswith(seed.roles[3].body.strip()) and all(p.body.strip() in text for p in seed.programs)
    with pytest.raises(G.GenomeError):
        G.instructions_for(seed, "janitor")


def _copy_seed(tmp_path):
    dst = tmp_path / "seed"
    shutil.copytree(G.seed_root(), dst, ignore=shutil.ignore_patterns("__pycache__", "*.py"))
    return dst


def test_loading_another_tree(tmp_path):
    root = _copy_seed(tmp_path)
    (root / "roles" / "director.md").write_text("custom director text")
    (root / "roles" / "archivist.md").write_text("an extra role")
    (root / "roles" / "tester.md").write_text("")                                         # an empty body still counts as present
    (root / "tools" / "notes.txt").write_text("not markdown")
    (root / "tools" / "grep.md").write_text("how to search")
    seed = G.load_seed(root)
    assert seed.roles[0].body == "custom director text" and G.role_names(seed) == G.ROLES + ("archivist",)   # required order, extras after
    assert "grep" in [t.name for t in seed.tools] and "notes" not in [t.name for t in seed.tools] and seed.root == root.resolve()
    assert G.load_seed().roles[0].body != "custom director text"                          # the default root is untouched


@pytest.mark.parametrize("missing", G.ROLES)
def test_a_missing_role_file_is_an_error(tmp_path, missing):
    root = _copy_seed(tmp_path)
    (root / "roles" / f"{missing}.md").unlink()
    with pytest.raises(G.GenomeError, match=missing):
        G.load_seed(root)
    partial = G.GenomeSeed(tuple(G.Entry(n, "x") for n in G.ROLES if n != missing), (), (), (), root)
    with pytest.raises(G.GenomeError, match=missing):
        G.require_roles(partial)
    assert G.role_names(partial) == tuple(n for n in G.ROLES if n != missing)


def test_missing_roots_and_optional_directories(tmp_path):
    with pytest.raises(G.GenomeError):
        G.load_seed(tmp_path / "nope")
    (tmp_path / "file").write_text("x")
    with pytest.raises(G.GenomeError):
        G.load_seed(tmp_path / "file")
    root = _copy_seed(tmp_path)
    shutil.rmtree(root / "tools")
    shutil.rmtree(root / "skills")
    seed = G.load_seed(root)
    assert seed.tools == () and seed.skills == ()
