"""Native programs on a GPU: the command-line benchmark in single-GPU emulation must verify every
element (#wrong = 0, exit status 0) for each collective, algorithm and dtype, and the smoke entry."""
import pytest

from conftest import run_native

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("args", [
    ["--collective", "all_reduce", "--nranks", "8"],
    ["--collective", "all_reduce", "--nranks", "8", "--algo", "ring"],
    ["--collective", "all_reduce", "--nranks", "4", "--dtype", "bf16", "--redop", "avg", "--data", "normal"],
    ["--collective", "all_reduce", "--nranks", "4", "--symmetric"],
    ["--collective", "reduce_scatter", "--nranks", "8", "--dtype", "fp16"],
    ["--collective", "all_gather", "--nranks", "8", "--algo", "ring"],
    ["--collective", "all_reduce", "--nranks", "4", "--transport", "shm"],
    ["--collective", "all_reduce", "--nranks", "4", "--graph"],
    ["--collective", "all_gather", "--nranks", "2", "--graph", "--symmetric"],
])
def test_bench_cli_verifies(native_build, args):
    proc = run_native("b200ccl_collective_bench", "--loopback", *args, "-b", "1024", "-e", "4194304", "-f", "64", "-w", "1", "-n",
                      "3", env={"B200CCL_WAIT_TIMEOUT_MS": "3000"})
    assert proc.returncode == 0, proc.stdout + proc.stderr
    rows = [l.split() for l in proc.stdout.splitlines() if l and not l.startswith("#")]
    assert len(rows) == 3 and all(r[9] == "0" for r in rows), proc.stdout


def test_public_api_program(native_build):
    proc = run_native("test_public_api", env={"B200CCL_WAIT_TIMEOUT_MS": "3000"})
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "public api ok" in proc.stdout


def test_smoke_entry():
    import __graft_entry__ as entry
    entry.smoke()
