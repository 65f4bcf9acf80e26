"""tokenizer / synth Python faces and the genome seed loader."""
import pytest

from prometheus_b200 import contracts, genome_seed, native, synth
from prometheus_b200 import tokenizer as T


def test_tokenizer_face(tmp_path):
    docs = ["the cat sat on the mat. the cat ate."] * 4 + ["a dog and a cat"]
    t = T.Tokenizer.train(docs, T.TrainConfig("tok-a", 300))
    ids = t.encode("the cat")
    assert t.decode(ids) == "the cat" and t.vocab_size == 300 and len(ids) < len("the cat")
    assert t.encode_grid([0, 9, 3]) == [T.FIRST_ARC, T.FIRST_ARC + 9, T.FIRST_ARC + 3]
    assert t.decode_bytes(t.encode_bytes(b"\xff\x00a")) == b"\xff\x00a"
    b, m = t.encode_batch(["the cat", "a"], add_bos=True, add_eos=True)
    assert b.shape == m.shape == (2, len(ids) + 2) and b[1, -1] == t.special_tokens["pad"] and m[1].sum() == 3
    assert t.encode_batch(["the cat"], max_len=2)[0].shape == (1, 2)
    t.freeze("2026-01-01T00:00:00Z")
    pointer = t.save(tmp_path / "tok")
    assert pointer["schema_id"] == "prometheus.vocab" and (tmp_path / "tok" / "vocab.jsonl").exists()
    contracts.validate(t.to_contract())
    contracts.validate(pointer)
    back = T.Tokenizer.load(tmp_path / "tok")
    assert back.encode("the cat") == ids and back.vocab_hash == t.vocab_hash and back.frozen
    with pytest.raises(T.TokenizerError):
        T.Tokenizer.train(docs, T.TrainConfig("x", 100))
    with pytest.raises(T.TokenizerError):
        T.Tokenizer.load(tmp_path / "missing")
    assert T.baseline_byte_tokens_per_word("ab cd") == 2.5 > 0


def test_synth_face_connects_engine_and_tokenizer():
    eng = native.serve.LocalEngine("m", 1, 2, 30000)
    gen = synth.engine_generator(eng)
    outs = gen(["a", "b", "c"], 3, 0.0)                       # three prompts through a batch limit of two
    assert len(outs) == 3 and outs[0] == eng.generate(["a"], 3, 0.0)[0][1]
    o = synth.Orchestrator(gen, max_tokens=4, styles=["news"])
    assert [r.style for r in o.rephrase_many([("d", "Cats purr.")])] == ["news"]
    t = T.Tokenizer.train(["x y z"] * 3, T.TrainConfig("g", 272))
    assert synth.grid_tokens(t, [[1, 2], [3, 4]]) == [261, 262, 263, 264]
    assert synth.STYLES[0] == "encyclopedia" and "math" in synth.DOMAINS
    assert synth.extract_answer("x\nAnswer: 7") == "7"


def test_genome_seed_loader(tmp_path):
    seed = genome_seed.load_seed()
    assert genome_seed.role_names(seed) == genome_seed.ROLES
    assert [p.name for p in seed.programs] == ["loop"] and seed.tools and seed.skills
    text = genome_seed.instructions_for(seed, "tester")
    assert text.startswith("# Tester") and "# Seed loop" in text
    with pytest.raises(genome_seed.GenomeError):
        genome_seed.instructions_for(seed, "overlord")
    (tmp_path / "roles").mkdir()
    (tmp_path / "roles" / "director.md").write_text("# D")
    with pytest.raises(genome_seed.GenomeError) as e:
        genome_seed.load_seed(tmp_path)
    assert "researcher" in str(e.value)
    with pytest.raises(genome_seed.GenomeError):
        genome_seed.load_seed(tmp_path / "nope")
    for r in genome_seed.ROLES[1:]:
        (tmp_path / "roles" / f"{r}.md").write_text(f"# {r}")
    (tmp_path / "roles" / "archivist.md").write_text("# extra")
    assert genome_seed.role_names(genome_seed.load_seed(tmp_path)) == genome_seed.ROLES + ("archivist",)
    # the kernel accepts the composed instructions
    k = native.kernel.Kernel(str(tmp_path / "ledger.jsonl"), str(tmp_path / "mirror"), str(tmp_path / "log"))
    (tmp_path / "mirror").mkdir(exist_ok=True)
    agent = k.spawn("director", genome_seed.instructions_for(seed, "director"), native.kernel.Quota(10, 1, 1), "loop")
    assert agent.depth == 0


def test_ci_checks(tmp_path):
    from prometheus_b200.utils import ci_checks

    assert ci_checks.main(["tree"]) == 0
    (tmp_path / "prometheus_b200").mkdir()
    (tmp_path / "prometheus_b200" / "bad.py").write_text("import os\nfrom tests import helper\n")
    assert ci_checks.check_test_imports(tmp_path) == ["production code imports tests/: prometheus_b200/bad.py"]
    junit = tmp_path / "j.xml"
    junit.write_text('<testsuite><testcase classname="a" name="ok"/>'
                     '<testcase classname="a" name="gpu"><skipped message="needs two GPUs"/></testcase>'
                     '<testcase classname="a" name="lazy"><skipped message="flaky, later"/></testcase></testsuite>')
    errs = ci_checks.check_skips(junit)
    assert len(errs) == 1 and "a::lazy" in errs[0] and ci_checks.main(["skips", str(junit)]) == 1
    assert ci_checks.main([]) == 2


def test_run_loop_on_cpu_with_overrides_and_spike_rollback():
    import io
    import json

    from prometheus_b200 import run

    out = io.StringIO()
    sets = ["batch=2", "seq_len=64", "n_docs=16", "vocab_size=512", "steps=4", "ckpt_every=2", "peak_lr=0.01"]
    res = run.run("tiny_fp32", sets, device="cpu", out=out)
    lines = [json.loads(l) for l in out.getvalue().splitlines()]
    assert [l["step"] for l in lines[:-1]] == [1, 2, 3, 4] and lines[-1]["summary"]["steps"] == 4
    assert res["summary"]["sequences_packed"] > 4 and res["summary"]["last_memory_checkpoint_step"] == 4
    assert all(h["loss"] == h["loss"] for h in res["history"])
    again = run.run("tiny_fp32", sets, device="cpu", out=io.StringIO())
    assert [h["loss"] for h in again["history"]] == [h["loss"] for h in res["history"]]     # deterministic loader + init
    with pytest.raises(ValueError):
        run.run("tiny_fp32", ["nonsense=1"], device="cpu", out=io.StringIO())
    with pytest.raises(ValueError):
        run.run("huge", [], device="cpu")
    cfg, tcfg, opts = run.apply_overrides(["fp8=true", "top_k=1", "softcap=20.0"], run.PRESETS["tiny_fp32"](),
                                          __import__("prometheus_b200").train.train_config_for(run.PRESETS["tiny_fp32"]()),
                                          run.RunOptions())
    assert opts.fp8 is True and cfg.top_k == 1 and tcfg.softcap == 20.0
    assert set(run.PRESETS) == {"tiny_fp32", "dense_1p3b", "moe_16b", "long_context", "latent"}


def test_bench_reference_arm_prints_the_unavailable_line():
    """`bench.py --impl reference` must exit 0 with one JSON line naming why the reference cannot
    run offline (jax is not installed here), never a fabricated number."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    res = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-500:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert ("unavailable" in line and isinstance(line["unavailable"], str) and line["unavailable"]) or "value" in line


def test_bench_argument_surface():
    """The flags the driver passes (and the extra configurations) parse."""
    import importlib.util
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    spec = importlib.util.spec_from_file_location("pb_bench_module", root / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    argv = sys.argv
    try:
        sys.argv = ["bench.py", "--gpus", "8", "--steps", "5", "--warmup", "3", "--config", "longctx"]
        a = mod.parse_args()
    finally:
        sys.argv = argv
    assert (a.gpus, a.steps, a.warmup, a.config, a.impl) == (8, 5, 3, "longctx", "ours")
