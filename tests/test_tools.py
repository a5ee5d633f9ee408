import json

import numpy as np
import pytest

from nexus_b200.lm.config import count_parameters, preset
from nexus_b200.tools import estimate as E
from nexus_b200.tools import tokenize as T


def test_parameter_counts_match_known_models():
    gpt2 = E.ModelShape.from_config(preset("gpt2-124m"))
    assert E.param_breakdown(gpt2)["total"] == 124_439_808 == count_parameters(preset("gpt2-124m"))
    llama = E.ModelShape(n_layer=32, d_model=4096, n_head=32, n_kv_head=32, d_ff=11008, vocab=32000, seq_len=4096,
                         learned_pos=0, tie_head=False, ffn_swiglu=True, bias=False, rmsnorm=True)
    assert E.param_breakdown(llama)["total"] == 6_738_415_616
    f = E.flops_per_token(gpt2)
    assert 6 * 85e6 < f < 6 * 124.4e6 + 12 * 12 * 768 * 1024


def test_memory_model_zero_stages_and_recompute():
    m = E.ModelShape.from_config(preset("gpt2-124m"), 1024, 16)
    dt = E.DTypePlan()
    base = E.memory_bytes(m, dt, E.Plan())
    n = 124_439_808
    assert base["static"] == n * (2 + 4 + 8 + 4)
    z = [E.memory_bytes(m, dt, E.Plan(dp=8, zero_stage=s))["static"] for s in range(4)]
    assert z[0] > z[1] > z[2] > z[3] and abs(z[3] - z[0] / 8) < 1
    assert E.memory_bytes(m, dt, E.Plan(full_recompute=True))["activations"] < 0.1 * base["activations"]
    assert E.memory_bytes(m, dt, E.Plan(flash_attention=False))["activations"] > base["activations"]
    assert E.memory_bytes(m, dt, E.Plan(tp=2))["activations"] == base["activations"] / 2


def test_step_time_and_auto_parallel():
    cl = E.Cluster()
    m = E.ModelShape.from_config(preset("gpt2-124m"), 1024, 16)
    t = E.step_time(m, E.Plan(), cl)
    assert 5e-3 < t["step_s"] < 50e-3 and t["tp_comm_s"] == 0 and abs(t["mfu"] - cl.mfu) < 1e-6
    assert E.step_time(m, E.Plan(tp=2), cl)["tp_comm_s"] > 0
    llama = E.ModelShape(n_layer=32, d_model=4096, n_head=32, n_kv_head=32, d_ff=11008, vocab=32000, seq_len=4096,
                         tie_head=False, ffn_swiglu=True, bias=False, rmsnorm=True)
    r = E.auto_parallel(llama, cl, E.AutoOptions(global_batch=64))
    assert r["feasible"] > 0 and len(r["best"]) == 3
    best = r["best"][0]
    assert best["dp"] * best["tp"] * best["pp"] * best["cp"] == 8 and best["memory_gib"] + cl.reserve_gib <= cl.mem_gib
    assert best["step_s"] <= r["best"][1]["step_s"]
    tight = E.auto_parallel(llama, E.Cluster(mem_gib=24.0), E.AutoOptions(global_batch=64))
    assert all(c["tp"] * c["pp"] > 1 or c["zero"] >= 1 for c in tight["best"])
    assert E.main(["--preset", "gpt2-124m", "--batch", "16", "--seq", "1024"]) == 0
    assert E.main(["--preset", "gpt2-124m", "--auto-parallel", "--global-batch", "64", "--json"]) == 0


def test_byte_bpe_and_shards(tmp_path):
    text = (b"the quick brown fox jumps over the lazy dog. " * 40) + "çığ öğe".encode()
    tok = T.ByteBpe.train(text, 300)
    assert 256 < tok.vocab_size <= 300
    ids = tok.encode(text)
    assert len(ids) < len(text) / 2 and tok.decode(ids) == text
    tok.save(str(tmp_path / "t.json"))
    again = T.ByteBpe.load(str(tmp_path / "t.json"))
    assert again.encode(b"the lazy fox") == tok.encode(b"the lazy fox")
    T.write_shard(str(tmp_path / "s.nxtk"), ids, tok.vocab_size)
    data, vocab = T.read_shard(str(tmp_path / "s.nxtk"))
    assert vocab == tok.vocab_size and data.dtype == np.uint16 and data.tolist() == ids
    (tmp_path / "c.txt").write_bytes(text)
    assert T.main(["train", "--vocab", "280", "--out", str(tmp_path / "t2.json"), str(tmp_path / "c.txt")]) == 0
    assert T.main(["encode", "--tokenizer", str(tmp_path / "t2.json"), "--out", str(tmp_path / "o.nxtk"), str(tmp_path / "c.txt")]) == 0
    with pytest.raises(ValueError):
        (tmp_path / "bad").write_bytes(b"XXXX" + b"\0" * 16)
        T.read_shard(str(tmp_path / "bad"))


def test_bench_evidence_rules(tmp_path):
    import sys
    from nexus_b200.bench import evidence as V
    ok = V.summarise([100, 101, 99, 100, 102], True, 100.0)
    assert ok["verdict"] == "ok" and ok["median"] == 100
    assert V.summarise([100, 150, 60, 100, 130], True, None)["verdict"].startswith("no-verdict")
    assert V.summarise([95, 96, 95, 96, 95], True, 100.0)["verdict"].startswith("regression")
    assert V.summarise([1.05, 1.05, 1.06], False, 1.0)["verdict"].startswith("regression")
    assert V.summarise([1.02, 1.02, 1.01], False, 1.0)["verdict"] == "ok"
    worker = tmp_path / "w.py"
    worker.write_text("import json, os; print('noise'); print(json.dumps({'value': [10.0, 10.1, 9.9]}))")
    r = V.sample_case("fake", [sys.executable, str(worker)], "value", 3, True, 10.0)
    assert r["samples"] == 9 and r["verdict"] == "ok"
    d = V.digests()
    assert any(k.endswith("gemm_sm100.cu") for k in d) and all(len(v) == 64 for v in d.values())
    ev = {"when": "t", "matrix": "kernels", "processes": 3, "warmup": 2, "samples": 3, "digests": d, "results": [r]}
    txt = V.report(ev)
    assert "| fake |" in txt and "verdict" in txt
    bad = tmp_path / "bad.py"
    bad.write_text("import sys; sys.exit(3)")
    with pytest.raises(RuntimeError):
        V.run_worker([sys.executable, str(bad)])


def test_docs_site_builds(tmp_path):
    """Every Markdown page under docs/ renders to an HTML page with the navigation and working relative links."""
    import os
    import re
    from pathlib import Path

    from nexus_b200.tools import site
    root = Path(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    files = site.build(root / "docs", tmp_path)
    names = {f.name for f in files}
    assert {"index.html", "kernels.html", "distributed.html"} <= names
    index = (tmp_path / "index.html").read_text()
    assert "<table>" in index and '<a href="kernels.html">' in index and "<nav>" in index
    for target in re.findall(r'href="([^"#:]+\.html)"', index):
        assert (tmp_path / target).exists(), target
    body, title = site.render_markdown("# T\n\ntext with `a*b*c` and *em* and [l](x.md#frag)\n\n```\n<raw>\n```\n\n1. one\n2. two\n")
    assert title == "T" and "<code>a*b*c</code>" in body and "<em>em</em>" in body
    assert 'href="x.html#frag"' in body and "&lt;raw&gt;" in body and "<ol><li>one</li><li>two</li></ol>" in body


@pytest.mark.parametrize("script,args", [("demo.py", []), ("dl_vision_classifier.py", []),
                                         ("hybrid_cluster_benchmark.py", []), ("lm_baseline.py", ["--json", "{tmp}/r.json"]),
                                         ("train_from_shards.py", ["--workdir", "{tmp}/shards"]),
                                         ("serve_demo.py", ["--small", "--requests", "6", "--max-new", "6", "--prompt-len", "12"]),
                                         ("custom_ops_showcase.py", [])])
def test_examples_run_on_cpu(tmp_path, script, args):
    """The example programs exit 0 on a machine without a GPU (each checks its own result)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "examples", script)] + [a.replace("{tmp}", str(tmp_path)) for a in args]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    if script == "lm_baseline.py":
        import json
        rep = json.load(open(tmp_path / "r.json"))
        assert rep["params_counted"] == rep["params_formula"] and rep["mfu"] is None and rep["tokens_per_second"] > 0


def test_parallel_bench_parameter_table_matches_the_model():
    """`bench.parallel` draws random weights from a (name, shape) table instead of building the model: the table
    must list exactly the parameters `lm.model.build` creates."""
    from nexus_b200.bench.parallel import build_meta
    from nexus_b200.lm.config import preset
    from nexus_b200.lm.model import build
    for name in ("llama2-7b", "gpt2-124m"):
        cfg = preset(name)
        cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 64, 4, 128, 96, 32
        if hasattr(cfg, "n_kv_head") and cfg.n_kv_head:
            cfg.n_kv_head = 4
        want = {n: tuple(p.shape) for n, p in build(cfg).named_parameters()}
        got = dict(build_meta(cfg))
        assert got == want


def test_estimate_core_is_native_and_ranked():
    from nexus_b200 import _native
    for name in ("estimate_params", "estimate_memory", "estimate_step_time", "estimate_evaluate", "estimate_auto_parallel"):
        assert hasattr(_native, name)
    big = E.ModelShape(n_layer=80, d_model=8192, n_head=64, n_kv_head=8, d_ff=28672, vocab=128256, seq_len=8192,
                       tie_head=False, ffn_swiglu=True, bias=False, rmsnorm=True)
    r = E.auto_parallel(big, E.Cluster(gpus=64), E.AutoOptions(top=8))
    assert 0 < r["feasible"] < r["tried"]
    keys = [(c["step_s"], c["tp"] * c["pp"] * c["cp"], c["zero"]) for c in r["best"]]
    assert keys == sorted(keys) and all(c["fits"] for c in r["best"])
    c0 = r["best"][0]
    again = E.evaluate(big, E.Cluster(gpus=64), c0["dp"], c0["tp"], c0["pp"], c0["cp"], c0["zero"], c0["micro_batch"],
                       c0["accum"], c0["recompute"])
    assert abs(again.step_s - c0["step_s"]) < 1e-12 and again.fits
    # hand-checked closed form of the static share: 18 bytes per parameter over tp*pp, ZeRO-3 divides all of it by dp
    n = E.param_breakdown(big)["total"]
    assert abs(again.static_gib * (1 << 30) - n * 18 / (c0["tp"] * c0["pp"]) / (c0["dp"] if c0["zero"] >= 3 else 1)) < \
        (1 << 20) or c0["zero"] in (1, 2)
