"""Native test programs that need no GPU: geometry, argument contract, rendezvous, NUMA."""
import pytest

from conftest import run_native

CPU_PROGRAMS = ["test_geometry", "test_validate", "test_bootstrap", "test_numa_topo", "test_socket_transport",
                "test_rdma_proxy", "test_timeline", "test_net_edges", "test_mpi_adapter", "test_ll_sim", "test_pipe_sim", "test_ibverbs_backend"]


@pytest.mark.parametrize("name", CPU_PROGRAMS)
def test_native_program(native_build, name):
    proc = run_native(name)
    assert proc.returncode == 0, f"{name} failed:\n{proc.stdout}\n{proc.stderr}"


def test_installed_package_is_usable_from_another_project(native_build, tmp_path):
    """cmake --install, then an outside project does find_package(b200ccl) and includes nano_nccl/*.h."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prefix, build = tmp_path / "prefix", tmp_path / "consumer_build"
    subprocess.run(["cmake", "--install", os.path.join(root, "build"), "--prefix", str(prefix)], check=True, capture_output=True)
    assert (prefix / "include" / "nano_nccl" / "communicator.h").exists() and (prefix / "lib" / "libb200ccl.so").exists()
    subprocess.run(["cmake", "-S", os.path.join(root, "tests", "cpp", "consumer"), "-B", str(build), "-G", "Ninja",
                    f"-DCMAKE_PREFIX_PATH={prefix}"], check=True, capture_output=True)
    subprocess.run(["ninja", "-C", str(build)], check=True, capture_output=True)
    env = dict(os.environ, LD_LIBRARY_PATH=str(prefix / "lib") + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    proc = subprocess.run([str(build / "app")], capture_output=True, text=True, env=env, timeout=120)
    assert proc.returncode == 0 and "consumer ok bf16 avg" in proc.stdout, proc.stdout + proc.stderr
