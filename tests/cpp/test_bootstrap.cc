// TCP rendezvous between real processes (fork): all-gather, barrier, error consensus and
// descriptor passing (a pipe written in one process is read through the descriptor received in
// another). No GPU needed.
#include "check.h"
#include "b200ccl/bootstrap.h"

#include <arpa/inet.h>
#include <cstring>
#include <netinet/in.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>
#include <vector>

using namespace b200ccl;

static int free_port() {
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    bind(fd, reinterpret_cast<sockaddr*>(&sa), sizeof(sa));
    socklen_t len = sizeof(sa);
    getsockname(fd, reinterpret_cast<sockaddr*>(&sa), &len);
    close(fd);
    return ntohs(sa.sin_port);
}

static int child(int rank, int size, int port) {
    auto bs = create_tcp_bootstrap("127.0.0.1", port, rank, size, 20000);
    T_CHECK(bs->rank() == rank && bs->size() == size);
    int mine = 100 + rank;
    std::vector<int> all(size);
    bs->allgather(&mine, all.data(), sizeof(int));
    for (int r = 0; r < size; ++r) T_CHECK(all[r] == 100 + r);
    bs->barrier();
    T_CHECK(bs->error_consensus("").empty());
    const std::string err = bs->error_consensus(rank == 1 ? "listener setup failed" : "");
    T_CHECK(err.find("process 1") != std::string::npos && err.find("listener setup failed") != std::string::npos);

    // Each process contributes the read end of a pipe that holds its rank, plus an absent entry.
    int p[2];
    T_CHECK(pipe(p) == 0);
    char tag = static_cast<char>('A' + rank);
    T_CHECK(write(p[1], &tag, 1) == 1);
    for (int round = 0; round < 2; ++round) {
        auto got = bs->exchange_fds({p[0], -1});
        T_CHECK(static_cast<int>(got.size()) == size);
        for (int r = 0; r < size; ++r) {
            T_CHECK(got[r].size() == 2 && got[r][0] >= 0 && got[r][1] == -1);
            close(got[r][0]);
        }
    }
    // Read rank (r+1)'s pipe through a received descriptor: only one reader per pipe.
    auto got = bs->exchange_fds({p[0]});
    const int from = (rank + 1) % size;
    char seen = 0;
    T_CHECK(read(got[from][0], &seen, 1) == 1 && seen == static_cast<char>('A' + from));
    for (auto& v : got) for (int fd : v) if (fd >= 0) close(fd);
    bs->barrier();
    return 0;
}

int main() {
    const int size = 4, port = free_port();
    std::vector<pid_t> pids;
    for (int r = 0; r < size; ++r) {
        const pid_t pid = fork();
        if (pid == 0) _exit(child(r, size, port));
        pids.push_back(pid);
    }
    int rc = 0;
    for (pid_t pid : pids) {
        int st = 0;
        waitpid(pid, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) rc = 1;
    }
    // size 1 needs no network at all
    auto solo = create_tcp_bootstrap("127.0.0.1", 1, 0, 1);
    int v = 5, w = 0;
    solo->allgather(&v, &w, sizeof(int));
    T_CHECK(w == 5);
    if (rc == 0) std::puts("bootstrap ok");
    return rc;
}
