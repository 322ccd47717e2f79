"""Native test programs that need no GPU: geometry, argument contract, rendezvous, NUMA."""
import pytest

from conftest import run_native

CPU_PROGRAMS = ["test_geometry", "test_validate", "test_bootstrap", "test_numa_topo", "test_socket_transport",
                "test_rdma_proxy", "test_timeline", "test_net_edges", "test_mpi_adapter", "test_ll_sim", "test_ibverbs_backend"]


@pytest.mark.parametrize("name", CPU_PROGRAMS)
def test_native_program(native_build, name):
    proc = run_native(name)
    assert proc.returncode == 0, f"{name} failed:\n{proc.stdout}\n{proc.stderr}"
