"""Data preparation, log checking and the lane launcher."""
import json

import numpy as np
import pytest

from cppmega_b200.data.indexed import read_index
from cppmega_b200.tools import data_prep, launch, log_check


def test_data_prep_writes_a_readable_indexed_dataset(tmp_path):
    src = tmp_path / "c.jsonl"
    docs = ["hello world, this is a document", "short", "another sufficiently long document for the corpus"]
    src.write_text("\n".join(json.dumps({"text": d}) for d in docs))
    out = str(tmp_path / "corpus")
    assert data_prep.main(["--input", str(src), "--tokenizer", "bytes", "--out", out, "--min-tokens", "8"]) == 0
    idx = read_index(out)
    assert idx["num_docs"] == 3 and len(idx["sizes"]) == 2                 # "short" was filtered out
    assert idx["dtype"] == np.uint16
    raw = np.fromfile(out + ".bin", dtype=np.uint16)
    first = raw[:idx["sizes"][0]]
    assert bytes(first[:-1].astype(np.uint8)).decode() == docs[0] and first[-1] == 256


def test_fim_transform_keeps_all_tokens():
    import random
    ids = list(range(10, 40))
    out = data_prep.fim_transform(ids, random.Random(1), 1.0, 1000, 1001, 1002)
    assert sorted(t for t in out if t < 1000) == ids and {1000, 1001, 1002} <= set(out)
    assert data_prep.fim_transform(ids, random.Random(1), 0.0, 1000, 1001, 1002) == ids


def _log(losses, fused="{'optimizer': True, 'moe': True}", fallbacks=None):
    lines = [f"[cppmega_b200] nam56r: 7.92B params (5.01B active), world 8 (dp8ep8), fused paths {fused}"]
    for i, l in enumerate(losses):
        rec = {"iteration": i + 1, "loss": l, "lm_loss": l, "tokens_per_s": 1000.0 + i, "elapsed_ms": 10.0}
        if fallbacks:
            rec["fallback_ops"] = fallbacks
        lines.append(json.dumps(rec))
    return "\n".join(lines)


def test_log_check_accepts_a_healthy_run_and_flags_bad_ones():
    good = log_check.parse_log(_log([10 - 0.3 * i for i in range(12)]))
    assert good.fused == {"optimizer": True, "moe": True}
    assert log_check.check(good, min_steps=10, require_fused=["moe", "optimizer"]) == []
    rising = log_check.parse_log(_log([5 + 0.3 * i for i in range(12)]))
    assert any("went up" in p for p in log_check.check(rising))
    nan = log_check.parse_log(_log([5.0, float("nan"), 4.0]))
    assert any("non-finite" in p for p in log_check.check(nan))
    fb = log_check.parse_log(_log([5.0, 4.0], fallbacks={"sparse_mla": 3}))
    assert any("fallbacks" in p for p in log_check.check(fb))
    assert any("not active" in p for p in log_check.check(log_check.parse_log(_log([5.0], fused="{'optimizer': False}")),
                                                          require_fused=["optimizer"]))
    cmp = log_check.compare(good, rising)
    assert cmp["tokens_per_s"]["b_over_a"] == pytest.approx(1.0) and cmp["loss_curve"]["steps"] == 12


def test_launch_lanes_render(capsys):
    assert launch.main(["list"]) == 0
    assert "b200_nam56r_bf16_ep8" in capsys.readouterr().out
    assert launch.main(["smoke_tiny", "--dry-run", "--set", "training.train_iters=3"]) == 0
    out = capsys.readouterr().out
    assert "torch.distributed.run" in out and "--train-iters 3" in out and "NCCL_NVLS_ENABLE=0" in out
    assert launch.main(["recipe:native_pretrain", "--dry-run", "--data", "/data/c"]) == 0
    assert "/data/c" in capsys.readouterr().out


def test_profile_report_groups_kernel_rows():
    from cppmega_b200.tools import profile_report as pr
    hdr = ("-" * 90 + "  " + "  ".join(["-" * 12] * 10) + "\n" +
           f"{'Name':>90}  " + "  ".join(f"{c:>12}" for c in ["Self CPU %", "Self CPU", "CPU total %", "CPU total", "CPU time avg",
                                                                "Self CUDA", "Self CUDA %", "CUDA total", "CUDA time avg", "# of Calls"]) + "\n")

    def row(name, self_cuda, calls):
        vals = ["0.00%", "0.000us", "0.00%", "0.000us", "0.000us", self_cuda, "1.00%", self_cuda, "1.000us", str(calls)]
        return f"{name[:90]:>90}  " + "  ".join(f"{v:>12}" for v in vals) + "\n"

    text = hdr + row("void cm::gemm_bf16_kernel<256, false, false, bf16, false, 0>(C", "100.000ms", 10) + \
        row("void cm::gemm_bf16_kernel<256, false, false, bf16, false, 1>(C", "20.000ms", 4) + \
        row("void cm::mimo::mimo_chunk_grad_kernel<128, 32>(CUtensorMap_st", "50.000ms", 13) + \
        row("LinearFnBackward", "100.000ms", 10) + \
        row("void at::native::vectorized_elementwise_kernel<8, at::native", "500.000us", 100) + \
        "Self CUDA time total: 170.5ms\n"
    rep = pr.report(text)
    groups = {g["group"]: g for g in rep["groups"]}
    assert abs(rep["total_ms"] - 170.5) < 1e-6                                     # the autograd row is not double counted
    assert groups["dense GEMM (tcgen05 bf16)"]["ms"] == 100.0 and groups["grouped GEMM (experts)"]["launches"] == 4
    assert groups["Mamba3 MIMO scan"]["ms"] == 50.0 and groups["PyTorch elementwise / copy / cat"]["ms"] == 0.5
    assert rep["top"][0]["ms"] == 100.0


def test_gpu_tool_modules_import_and_list_their_cases():
    """The GPU-side tools must at least import on a CPU box and expose the cases the profile notes cite."""
    from cppmega_b200.tools import kernel_bench, moe_bench, ncu_cases
    for name in ("gemm", "scan_fwd", "scan_bwd", "m2rnn_bwd", "sparse_mla", "indexer", "mxfp8_gemm", "adamw", "rmsnorm",
                 "rmsnorm_bwd", "quantize", "strided_copy", "moe_local", "ce"):
        assert name in ncu_cases.CASES, name
    for name in ("gemm", "grouped", "rmsnorm", "ce", "scan", "mxfp8_gemm", "longctx"):
        assert name in kernel_bench.CASES, name
    assert callable(moe_bench.main)
    from cppmega_b200.tools import kernel_bench_reference
    assert set(kernel_bench_reference.CASES) == {"m2rnn", "sparse_mla", "indexer", "linear_ce", "gemm"}
    assert kernel_bench_reference.main([]) == 2
    pk = kernel_bench.peaks()
    assert pk["bf16_tflops"] > 0 and pk["kind"] in ("measured", "fallback")


def test_verify_dataset_accepts_good_and_flags_bad(tmp_path):
    import numpy as np
    from cppmega_b200.data.indexed import write_indexed_dataset
    from cppmega_b200.tools import verify_dataset
    docs = [np.array([5, 6, 7, 0], dtype=np.int32), np.array([9, 0], dtype=np.int32)]
    prefix = str(tmp_path / "d")
    write_indexed_dataset(prefix, docs, dtype=np.int32)
    good = verify_dataset.verify(prefix, vocab_size=16, eod=0)
    assert good["problems"] == [] and good["documents"] == 2 and good["tokens"] == 6
    assert any("vocabulary" in p for p in verify_dataset.verify(prefix, vocab_size=8)["problems"])
    assert any("eod" in p for p in verify_dataset.verify(prefix, eod=3)["problems"])
    with open(prefix + ".bin", "ab") as f:
        f.write(b"\\x00\\x00\\x00\\x00")
    assert any(".bin file" in p for p in verify_dataset.verify(prefix)["problems"])
    assert verify_dataset.main([prefix]) == 1


def test_nan_hunter_names_the_first_bad_module():
    import torch
    import torch.nn as nn
    from cppmega_b200.utils.nan_hunt import NonFiniteHunter

    class Bad(nn.Module):
        def forward(self, x):
            return x / (x - x)            # 0 / 0

    net = nn.Sequential(nn.Linear(4, 4), nn.Tanh(), Bad(), nn.Linear(4, 2))
    with NonFiniteHunter(net) as h:
        net(torch.ones(3, 4)).sum().backward()
        assert h.first == ("forward", "2") and "forward of '2'" in h.report()
        h.reset()
        net[2] = nn.Identity()
    with NonFiniteHunter(net) as h2:
        net(torch.ones(3, 4)).sum().backward()
        assert h2.first is None and "finite" in h2.report()


def test_dashboard_discovers_runs_and_renders_them():
    """Two fake runs publish records on their metrics endpoints; the dashboard finds them, computes the analytics and
    serves the overview, the detail page and the JSON API."""
    import json as _json
    import urllib.request
    from cppmega_b200.tools.dashboard import Dashboard, analytics
    from cppmega_b200.utils.monitor import MetricsServer
    servers = [MetricsServer(0).start() for _ in range(2)]
    try:
        for k, s in enumerate(servers):
            for it in range(1, 9):
                s.publish({"iteration": it, "loss": 10.0 - 0.5 * it - k, "grad_norm": 1.0, "elapsed_ms": 100.0 + it,
                           "tokens_per_s": 1000.0 * (k + 1), "tflops_per_gpu": 400.0})
        ports = [s.port for s in servers]
        dash = Dashboard("127.0.0.1", ports + [1], 0).serve(block=False)       # port 1: nothing listens there
        import threading
        t = threading.Thread(target=dash._httpd.serve_forever, daemon=True)
        t.start()
        try:
            base = f"http://127.0.0.1:{dash.listen[1]}"
            runs = _json.loads(urllib.request.urlopen(base + "/api/runs", timeout=5).read())
            assert sorted(r["port"] for r in runs) == sorted(ports)
            a = runs[0]["analytics"]
            assert a["records"] == 8 and a["loss_slope_per_iteration"] < 0 and a["median_tokens_per_s"] in (1000.0, 2000.0)
            page = urllib.request.urlopen(base + "/", timeout=5).read().decode()
            assert all(str(p) in page for p in ports) and "<svg" in page
            detail = urllib.request.urlopen(f"{base}/run/{ports[0]}", timeout=5).read().decode()
            assert "loss_slope_per_iteration" in detail and "tokens/s" in detail
        finally:
            dash.stop()
    finally:
        for s in servers:
            s.stop()
    assert analytics([])["records"] == 0


def test_supervised_launch_resumes_from_the_last_checkpoint_after_a_rank_failure(tmp_path, capfd):
    """Host-side fault injection on two gloo ranks: the last rank raises after iteration 3 of a fresh run; the supervisor
    starts the job again with ``--load`` and it finishes from the checkpoint of iteration 2."""
    import socket
    from cppmega_b200.checkpoint import sharded
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    save = str(tmp_path / "ckpt")
    rc = launch.main(["smoke_tiny", "--max-restarts", "2", "--master-port", str(port),
                      "--set", "training.train_iters=6", "--set", f"training.save={save}", "--set", "training.save_interval=2",
                      "--extra", "--inject-failure-at-iteration", "3"])
    out = capfd.readouterr().out
    assert rc == 0, out[-2000:]
    assert "restarting from iteration 2" in out
    assert sharded.latest_iteration(save) == 6


def test_supervisor_gives_up_after_the_allowed_restarts():
    calls = []

    def run(cmd):
        calls.append(cmd)
        return 7

    rc = launch.supervise(["--save", "/nonexistent/ckpt"], 1, 29500, 2, run=run)
    assert rc == 7 and len(calls) == 3
    assert all("--load" not in c for c in calls)                 # nothing was ever saved: every attempt starts fresh
    ports = [c[c.index("--master-port") + 1] if "--master-port" in c else None for c in calls]
    assert ports == [None, None, None]                           # one process: plain python, no rendezvous


def test_tp_bench_needs_ranks_and_knows_the_recipe_shapes(capsys):
    from cppmega_b200.tools import tp_bench
    assert tp_bench.main([]) == 0
    assert '"unavailable"' in capsys.readouterr().out
    shapes = {name: (kind, k, n) for name, kind, k, n in tp_bench._shapes()}
    assert shapes["mamba_in_proj"] == ("ag_gemm", 4096, 24960) and shapes["mamba_out_proj"] == ("gemm_rs", 8192, 4096)
