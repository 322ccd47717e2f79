"""The result renderer and the RDMA mode A/B driver, as far as they go without a GPU."""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_tool(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "bench", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_render_single_and_comparison(tmp_path):
    tool = load_tool("render_performance_md")
    ours = [{"collective": "all_reduce", "algo": "nvls", "bytes": 1 << 20, "time_us": 12.5, "algbw_gbs": 83.9, "busbw_gbs": 146.8, "wrong": 0},
            {"collective": "all_reduce", "algo": "oneshot", "bytes": 1024, "time_us": 9.8, "algbw_gbs": 0.1, "busbw_gbs": 0.18, "wrong": 0}]
    (tmp_path / "ours.json").write_text(json.dumps(ours))
    md = tool.render([str(tmp_path / "ours.json")], "AllReduce")
    lines = md.splitlines()
    assert lines[0] == "## AllReduce" and "#wrong" in lines[2]
    assert lines[4].startswith("| 1 KiB | oneshot | 9.80") and lines[5].startswith("| 1 MiB | nvls | 12.50")
    # bench.py line with a sweep, in a log with other text around it
    line = {"metric": "allreduce_busbw", "value": 700.0, "ms_per_step": 0.16, "config": {"bytes": 1 << 26},
            "sweep": [{"bytes": 1 << 20, "time_us": 20.0, "busbw_gbs": 91.75}, {"bytes": 1 << 26, "time_us": 160.0, "busbw_gbs": 734.0}]}
    (tmp_path / "nccl.log").write_text("warming up\n" + json.dumps(line) + "\n")
    md = tool.render([f"ours={tmp_path / 'ours.json'}", f"nccl={tmp_path / 'nccl.log'}"])
    assert "| size | ours busbw (GB/s) | nccl busbw (GB/s) | ours / nccl |" in md
    assert "| 1 MiB | 146.80 | 91.75 | 1.60 |" in md and "| 64 MiB | – | 734.00 | – |" in md
    # tuner table: the winners per size
    tuner = {"rows": ours, "best": ours[:1], "n_gpus": 8}
    (tmp_path / "tuner.json").write_text(json.dumps(tuner))
    assert tool.render([str(tmp_path / "tuner.json")]).count("\n") == 3
    assert tool.human(3 << 30) == "3 GiB" and tool.human(1500) == "1500 B"


def test_rdma_ab_parsing_summary_and_dry_run(tmp_path, capsys):
    tool = load_tool("rdma_modes_ab")
    table = """# b200ccl collective_bench
#           algo    dtype    redop  transport      size(B)        count   time(us)      algbw      busbw   #wrong      max_abs
            ring    float      sum       rdma      1048576       262144      97.06      10.80      18.91        0  9.53674e-07
            ring    float      sum       rdma      4194304      1048576     300.00      13.98      24.47        0  9.53674e-07
"""
    assert tool.parse_table(table) == [(1048576, 97.06, 18.91, 0), (4194304, 300.0, 24.47, 0)]
    rows = tool.summarise({"send-shared": {1048576: [18.0, 19.0, 17.0]}, "write-shared": {1048576: [20.0]}})
    assert rows[0] == {"mode": "send-shared", "bytes": 1048576, "runs": 3, "best_gbs": 19.0, "median_gbs": 18.0, "worst_gbs": 17.0}
    md = tool.markdown(rows)
    assert "send-shared median (best) GB/s" in md and "| 1048576 | 18.00 (19.00) | 20.00 (20.00) |" in md
    rc = tool.main(["--out-dir", str(tmp_path / "ab"), "--runs", "1", "--modes", "write-shared,send-dedicated-gdr", "--nranks", "4",
                    "--loopback", "--dry-run"])
    out = capsys.readouterr().out.splitlines()
    assert rc == 0 and len(out) == 2
    assert "B200CCL_RDMA_USE_WRITE=1" in out[0] and "B200CCL_RDMA_SHARED_PROGRESS=1" in out[0] and "--transport rdma" in out[0]
    assert "B200CCL_RDMA_GDR=1" in out[1] and "--nranks 4 --loopback" in out[1]


def test_native_multi_process_benchmark_agrees_on_a_setup_failure():
    # Two processes of the command-line benchmark on a machine without a GPU: the communicator cannot
    # be created, every process learns of it through the rendezvous and all leave with the same status
    # instead of one waiting for the other.
    import socket
    import subprocess
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    binary = os.path.join(root, "build", "bin", "b200ccl_collective_bench")
    if not os.path.exists(binary):
        pytest.skip("native benchmark not built")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    procs = [subprocess.Popen([binary, "--world", "2", "--rank", str(r), "--addr", f"127.0.0.1:{port}", "-b", "1024", "-e", "1024"],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [(p.wait(timeout=120), p.stdout.read()) for p in procs]
    assert [rc for rc, _ in outs] == [3, 3], outs
    assert all("communicator setup failed" in out for _, out in outs), outs


def test_bench_py_traffic_model_and_median():
    # bench.py's per-direction NVLink byte model (link_fraction_of_900) and its batch statistics
    spec = importlib.util.spec_from_file_location("bench_main", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    S = 64 << 20
    assert bench.link_bytes_per_direction("nvls", S, 8) == S * 1.125       # own shard out once + the result back, self included
    assert bench.link_bytes_per_direction("twoshot", S, 8) == S * 1.75     # pull 7/8, push 7/8
    assert bench.link_bytes_per_direction("twoshot", S, 2) == S
    assert bench.link_bytes_per_direction("oneshot", S, 4) == 3 * S
    assert bench.link_bytes_per_direction("ll", 1024, 8) == 2 * 1024 * 7   # 8 bytes on the wire per 4 of data
    assert bench.link_bytes_per_direction("copy", S, 1) == 0
    assert bench.busbw(S, 1e-3, 8) == S / 1e-3 / 1e9 * 1.75 and bench.busbw(S, 1e-3, 1) == S / 1e-3 / 1e9
    assert bench.median([3.0, 1.0, 2.0]) == 2.0 and bench.median([4.0, 1.0, 2.0, 3.0]) == 2.5
    peak, kind = bench.measured_peaks()
    assert peak > 1000 and kind in ("measured", "fallback")
