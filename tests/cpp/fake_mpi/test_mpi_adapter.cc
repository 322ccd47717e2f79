// The MPI adapter of the control plane (src/bootstrap/mpi/mpi_bootstrap.cc), compiled against the
// in-process stand-in of this folder: four thread-ranks check rank/size, all-gather, barrier,
// error consensus (the reference's MPI_Allreduce(MIN) + gather of messages,
// src/collective/all_reduce/mpi_communicator.cc:38-75), descriptor passing over AF_UNIX sockets
// named through the adapter's own all-gather, a failing MPI call turned into an exception that
// names it, and the refusal to start before MPI_Init / after MPI_Finalize. No GPU, no MPI.
#include "../check.h"
#include "b200ccl/mpi.h"

#include <atomic>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

using namespace b200ccl;

static std::atomic<int> g_failures{0};

static void rank_main(MPI_Comm world, int rank, int size) {
    fake_mpi_bind_thread(world, rank);
    try {
        auto bs = create_mpi_bootstrap(world);
        T_CHECK(bs->rank() == rank && bs->size() == size);
        long mine = 1000 + rank;
        std::vector<long> all(size);
        bs->allgather(&mine, all.data(), sizeof(long));
        for (int r = 0; r < size; ++r) T_CHECK(all[r] == 1000 + r);
        bs->barrier();
        T_CHECK(bs->error_consensus("").empty());
        const std::string err = bs->error_consensus(rank == 2 ? "socket listener setup failed" : "");
        T_CHECK(err.find("process 2") != std::string::npos && err.find("listener setup failed") != std::string::npos);

        // Descriptor passing: each rank offers the read end of a pipe holding its tag.
        int p[2];
        T_CHECK(pipe(p) == 0);
        char tag = static_cast<char>('a' + rank);
        T_CHECK(write(p[1], &tag, 1) == 1);
        for (int round = 0; round < 2; ++round) {
            auto got = bs->exchange_fds({p[0], -1});
            T_CHECK(static_cast<int>(got.size()) == size);
            for (int r = 0; r < size; ++r) {
                T_CHECK(got[r].size() == 2 && got[r][0] >= 0 && got[r][1] == -1);
                if (round == 1 && r == (rank + 1) % size) {
                    char seen = 0;
                    T_CHECK(read(got[r][0], &seen, 1) == 1 && seen == static_cast<char>('a' + r));
                }
                close(got[r][0]);
            }
        }
        close(p[0]);
        close(p[1]);

        // A failing MPI call becomes an exception that names the call (every rank sees the failure).
        bs->barrier();
        if (rank == 0) fake_mpi_fail_next_allgather(world, MPI_ERR_OTHER);
        bs->barrier();
        bool threw = false;
        try {
            bs->allgather(&mine, all.data(), sizeof(long));
        } catch (const std::exception& e) {
            threw = std::string(e.what()).find("MPI_Allgather failed") != std::string::npos;
        }
        T_CHECK(threw);
        bs->allgather(&mine, all.data(), sizeof(long));  // and the next one works again
        T_CHECK(all[size - 1] == 1000 + size - 1);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "rank %d: %s\n", rank, e.what());
        g_failures.fetch_add(1);
    }
}

int main() {
    const int size = 4;
    MPI_Comm world = fake_mpi_create_world(size);
    std::vector<std::thread> threads;
    for (int r = 0; r < size; ++r) threads.emplace_back(rank_main, world, r, size);
    for (auto& t : threads) t.join();
    T_CHECK(g_failures.load() == 0);

    // One rank alone: no sockets are needed, descriptors are duplicated locally.
    MPI_Comm solo = fake_mpi_create_world(1);
    fake_mpi_bind_thread(solo, 0);
    {
        auto bs = create_mpi_bootstrap(solo);
        auto got = bs->exchange_fds({0});
        T_CHECK(got.size() == 1 && got[0].size() == 1 && got[0][0] >= 0 && got[0][0] != 0);
        close(got[0][0]);
    }
    // Not initialised, or already finalised: refused with a message.
    for (int mode = 0; mode < 2; ++mode) {
        fake_mpi_set_initialized(mode == 0 ? 0 : 1, mode == 0 ? 0 : 1);
        bool threw = false;
        try {
            create_mpi_bootstrap(solo);
        } catch (const std::exception& e) {
            threw = std::string(e.what()).find("initialised") != std::string::npos;
        }
        T_CHECK(threw);
    }
    fake_mpi_set_initialized(1, 0);
    fake_mpi_destroy_world(solo);
    fake_mpi_destroy_world(world);
    std::printf("mpi adapter ok\n");
    return 0;
}
