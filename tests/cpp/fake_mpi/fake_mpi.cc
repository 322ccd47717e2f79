// See mpi.h in this folder: thread-ranks, one shared buffer, a generation barrier.
#include "mpi.h"

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

struct FakeMpiWorld {
    int size = 1;
    std::mutex mu;
    std::condition_variable cv;
    int arrived = 0;
    unsigned long generation = 0;
    std::vector<char> gather;
    std::atomic<int> fail_allgather{0};
    int fail_left = 0;
};

namespace {

thread_local FakeMpiWorld* t_world = nullptr;
thread_local int t_rank = -1;
std::atomic<int> g_initialized{1}, g_finalized{0};

std::size_t type_size(MPI_Datatype t) { return t == MPI_INT ? sizeof(int) : 1; }

// All ranks meet; `last` runs in exactly one of them (under the lock) once everyone has arrived.
template <typename F>
void meet(FakeMpiWorld* w, F last) {
    std::unique_lock<std::mutex> lock(w->mu);
    const unsigned long gen = w->generation;
    if (++w->arrived == w->size) {
        last();
        w->arrived = 0;
        ++w->generation;
        w->cv.notify_all();
    } else {
        w->cv.wait(lock, [&] { return w->generation != gen; });
    }
}

}  // namespace

extern "C" {

int MPI_Initialized(int* flag) { *flag = g_initialized.load(); return MPI_SUCCESS; }
int MPI_Finalized(int* flag) { *flag = g_finalized.load(); return MPI_SUCCESS; }

int MPI_Comm_rank(MPI_Comm comm, int* rank) {
    if (comm == nullptr || comm != t_world) return MPI_ERR_OTHER;
    *rank = t_rank;
    return MPI_SUCCESS;
}

int MPI_Comm_size(MPI_Comm comm, int* size) {
    if (comm == nullptr) return MPI_ERR_OTHER;
    *size = comm->size;
    return MPI_SUCCESS;
}

int MPI_Allgather(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                  MPI_Datatype recvtype, MPI_Comm comm) {
    if (comm == nullptr || comm != t_world) return MPI_ERR_OTHER;
    const std::size_t bytes = static_cast<std::size_t>(sendcount) * type_size(sendtype);
    if (bytes != static_cast<std::size_t>(recvcount) * type_size(recvtype)) return MPI_ERR_OTHER;
    {
        std::lock_guard<std::mutex> lock(comm->mu);
        if (comm->gather.size() < bytes * comm->size) comm->gather.resize(bytes * comm->size);
        std::memcpy(comm->gather.data() + bytes * t_rank, sendbuf, bytes);
    }
    int code = MPI_SUCCESS;
    meet(comm, [&] {
        if (comm->fail_allgather.load() != 0) comm->fail_left = comm->size;
    });
    {
        std::lock_guard<std::mutex> lock(comm->mu);
        if (comm->fail_left > 0) {
            code = comm->fail_allgather.load();
            if (--comm->fail_left == 0) comm->fail_allgather.store(0);
        } else {
            std::memcpy(recvbuf, comm->gather.data(), bytes * comm->size);
        }
    }
    meet(comm, [] {});  // nobody overwrites the shared buffer while a peer still copies from it
    return code;
}

int MPI_Barrier(MPI_Comm comm) {
    if (comm == nullptr || comm != t_world) return MPI_ERR_OTHER;
    meet(comm, [] {});
    return MPI_SUCCESS;
}

int MPI_Error_string(int errorcode, char* string, int* resultlen) {
    *resultlen = std::snprintf(string, MPI_MAX_ERROR_STRING, "fake MPI error %d", errorcode);
    return MPI_SUCCESS;
}

MPI_Comm fake_mpi_create_world(int size) {
    FakeMpiWorld* w = new FakeMpiWorld;
    w->size = size;
    return w;
}
void fake_mpi_destroy_world(MPI_Comm world) { delete world; }
void fake_mpi_bind_thread(MPI_Comm world, int rank) {
    t_world = world;
    t_rank = rank;
}
void fake_mpi_set_initialized(int initialized, int finalized) {
    g_initialized.store(initialized);
    g_finalized.store(finalized);
}
void fake_mpi_fail_next_allgather(MPI_Comm world, int code) { world->fail_allgather.store(code); }

}  // extern "C"
