// libibverbs implementation of VerbsBackend. Part of the library only with B200CCL_ENABLE_RDMA_VERBS=ON.
// Where libibverbs is not installed it is still compiled and run by
// tests/cpp/fake_ibverbs/test_ibverbs_backend.cc against a stand-in header with an in-process loopback
// fabric (no HCA); it has not been run on real hardware.
//
// Parity: nano-nccl src/transport/rdma/rdma_endpoint.cc:27-37, 41-80, 164-248 (device choice by
// interface name through sysfs or by GID == the interface's IPv6/IPv4-mapped address, port 1 must be
// ACTIVE, GID index from the environment, one context + protection domain, allocate_cq),
// rdma_qp.cc:30-195 (RC queue pair on one shared CQ, sq_sig_all = 0, max_inline_data = 64,
// INIT → RTR with path MTU = min(local, remote), GRH when the port is Ethernet, min_rnr_timer 12 →
// RTS with timeout 14, retry_cnt 7, rnr_retry 7), rdma_gdr.cc:112-136 (dma-buf registration with a
// fallback to peer-memory ibv_reg_mr; never a silent host fallback).
#if defined(B200CCL_ENABLE_RDMA_VERBS)

#include "core/env.h"
#include "mem/cu_driver.h"
#include "transport/rdma/verbs_backend.h"

#include <infiniband/verbs.h>

#include <arpa/inet.h>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>
#include <unistd.h>

namespace b200ccl::transport::rdma {

namespace {

constexpr std::uint8_t kPort = 1;

struct Context {
    ibv_context* ctx = nullptr;
    ibv_pd* pd = nullptr;
    ibv_port_attr port{};
    int gid_index = 0;
    ibv_gid gid{};
    ~Context() {
        if (pd) ibv_dealloc_pd(pd);
        if (ctx) ibv_close_device(ctx);
    }
};

bool device_serves_interface(const char* hca, const std::string& ifname) {
    if (ifname.empty()) return true;
    std::ifstream probe(std::string("/sys/class/infiniband/") + hca + "/device/net/" + ifname + "/ifindex");
    return probe.good();
}

std::shared_ptr<Context> open_context() {
    const std::string ifname = env::get_string("B200CCL_RDMA_IFNAME", "", "NANO_NCCL_RDMA_IFNAME");
    const int gid_index = static_cast<int>(env::get_int("B200CCL_RDMA_GID_INDEX", 0, "NANO_NCCL_RDMA_GID_INDEX"));
    int count = 0;
    ibv_device** list = ibv_get_device_list(&count);
    if (!list || count == 0) throw std::runtime_error("rdma: no RDMA device found");
    auto out = std::make_shared<Context>();
    std::string why = "no device matches interface '" + ifname + "'";
    for (int i = 0; i < count && !out->ctx; ++i) {
        if (!device_serves_interface(ibv_get_device_name(list[i]), ifname)) continue;
        ibv_context* ctx = ibv_open_device(list[i]);
        if (!ctx) continue;
        ibv_port_attr attr{};
        if (ibv_query_port(ctx, kPort, &attr) != 0 || attr.state != IBV_PORT_ACTIVE) {
            why = std::string(ibv_get_device_name(list[i])) + " port 1 is not ACTIVE";
            ibv_close_device(ctx);
            continue;
        }
        out->ctx = ctx;
        out->port = attr;
    }
    ibv_free_device_list(list);
    if (!out->ctx) throw std::runtime_error("rdma: " + why);
    out->gid_index = gid_index;
    if (ibv_query_gid(out->ctx, kPort, gid_index, &out->gid) != 0) throw std::runtime_error("rdma: ibv_query_gid failed");
    out->pd = ibv_alloc_pd(out->ctx);
    if (!out->pd) throw std::runtime_error("rdma: ibv_alloc_pd failed");
    return out;
}

struct IbCq : CompletionQueue {
    ibv_cq* cq = nullptr;
    ~IbCq() override { if (cq) ibv_destroy_cq(cq); }
    int poll(int max_entries, Completion* out) override {
        ibv_wc wc[32];
        const int want = max_entries < 32 ? max_entries : 32;
        const int n = ibv_poll_cq(cq, want, wc);
        for (int i = 0; i < n; ++i) {
            out[i].wr_id = wc[i].wr_id;
            out[i].status = wc[i].status == IBV_WC_SUCCESS ? 0 : static_cast<int>(wc[i].status);
            out[i].byte_len = wc[i].byte_len;
            out[i].imm = (wc[i].wc_flags & IBV_WC_WITH_IMM) ? ntohl(wc[i].imm_data) : 0;
            switch (wc[i].opcode) {
                case IBV_WC_SEND: out[i].opcode = WcOpcode::Send; break;
                case IBV_WC_RDMA_WRITE: out[i].opcode = WcOpcode::RdmaWrite; break;
                case IBV_WC_RECV_RDMA_WITH_IMM: out[i].opcode = WcOpcode::RecvRdmaWithImm; break;
                default: out[i].opcode = WcOpcode::Recv; break;
            }
        }
        return n;
    }
};

struct IbQp : QueuePair {
    std::shared_ptr<Context> c;
    ibv_qp* qp = nullptr;
    std::uint32_t psn = 0;
    ~IbQp() override { if (qp) ibv_destroy_qp(qp); }

    void fill_local_info(RdmaPeerInfo* info) const override {
        info->qpn = qp->qp_num;
        info->psn = psn;
        info->lid = c->port.lid;
        info->gid_index = static_cast<std::uint8_t>(c->gid_index);
        info->active_mtu = static_cast<std::uint8_t>(c->port.active_mtu);
        std::memcpy(info->gid, c->gid.raw, 16);
    }

    void connect(const RdmaPeerInfo& remote) override {
        ibv_qp_attr a{};
        a.qp_state = IBV_QPS_INIT;
        a.pkey_index = 0;
        a.port_num = kPort;
        a.qp_access_flags = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE;
        if (ibv_modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) != 0)
            throw std::runtime_error("rdma: queue pair INIT failed");
        std::memset(&a, 0, sizeof(a));
        a.qp_state = IBV_QPS_RTR;
        a.path_mtu = static_cast<ibv_mtu>(negotiate_path_mtu(static_cast<std::uint8_t>(c->port.active_mtu), remote.active_mtu));
        a.dest_qp_num = remote.qpn;
        a.rq_psn = remote.psn;
        a.max_dest_rd_atomic = 1;
        a.min_rnr_timer = 12;
        a.ah_attr.port_num = kPort;
        a.ah_attr.dlid = remote.lid;
        if (c->port.link_layer == IBV_LINK_LAYER_ETHERNET || remote.lid == 0) {
            a.ah_attr.is_global = 1;
            std::memcpy(a.ah_attr.grh.dgid.raw, remote.gid, 16);
            a.ah_attr.grh.sgid_index = static_cast<std::uint8_t>(c->gid_index);
            a.ah_attr.grh.hop_limit = 1;
        }
        if (ibv_modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN |
                                      IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER) != 0)
            throw std::runtime_error("rdma: queue pair RTR failed");
        std::memset(&a, 0, sizeof(a));
        a.qp_state = IBV_QPS_RTS;
        a.timeout = 14;
        a.retry_cnt = 7;
        a.rnr_retry = 7;
        a.sq_psn = psn;
        a.max_rd_atomic = 1;
        if (ibv_modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN |
                                      IBV_QP_MAX_QP_RD_ATOMIC) != 0)
            throw std::runtime_error("rdma: queue pair RTS failed");
    }

    void post_send(const SendWr& wr) override {
        ibv_sge sge{};
        sge.addr = reinterpret_cast<std::uint64_t>(wr.local_addr);  // straight from the FIFO slot: no bounce copy
        sge.length = wr.length;
        sge.lkey = wr.lkey;
        ibv_send_wr w{};
        w.wr_id = wr.wr_id;
        w.sg_list = &sge;
        w.num_sge = wr.length ? 1 : 0;
        w.send_flags = (wr.signaled ? IBV_SEND_SIGNALED : 0) | (wr.inline_data ? IBV_SEND_INLINE : 0);
        switch (wr.opcode) {
            case WrOpcode::Send: w.opcode = IBV_WR_SEND; break;
            case WrOpcode::RdmaWrite: w.opcode = IBV_WR_RDMA_WRITE; break;
            case WrOpcode::RdmaWriteWithImm: w.opcode = IBV_WR_RDMA_WRITE_WITH_IMM; w.imm_data = htonl(wr.imm); break;
        }
        w.wr.rdma.remote_addr = wr.remote_addr;
        w.wr.rdma.rkey = wr.rkey;
        ibv_send_wr* bad = nullptr;
        if (ibv_post_send(qp, &w, &bad) != 0) throw std::runtime_error("rdma: ibv_post_send failed");
    }

    void post_recv(const RecvWr& wr) override {
        ibv_sge sge{};
        sge.addr = reinterpret_cast<std::uint64_t>(wr.addr);
        sge.length = wr.length;
        sge.lkey = wr.lkey;
        ibv_recv_wr w{};
        w.wr_id = wr.wr_id;
        w.sg_list = &sge;
        w.num_sge = 1;
        ibv_recv_wr* bad = nullptr;
        if (ibv_post_recv(qp, &w, &bad) != 0) throw std::runtime_error("rdma: ibv_post_recv failed");
    }
};

class IbVerbs final : public VerbsBackend {
public:
    IbVerbs() : c_(open_context()) {}
    std::string name() const override { return "ibverbs"; }

    MemoryRegion register_memory(void* addr, std::size_t length) override {
        ibv_mr* mr = ibv_reg_mr(c_->pd, addr, length, IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE);
        if (!mr) throw std::runtime_error("rdma: ibv_reg_mr failed");
        return MemoryRegion{addr, length, mr->lkey, mr->rkey, reinterpret_cast<std::uint64_t>(mr)};
    }

    MemoryRegion register_device_memory(void* addr, std::size_t length) override {
        const int access = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE;
        ibv_mr* mr = nullptr;
#if defined(CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD)
        // dma-buf export of the device range, where the driver and the kernel offer it.
        using GetHandle = CUresult (*)(void*, CUdeviceptr, size_t, CUmemRangeHandleType, unsigned long long);
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetHandleForAddressRange", &fn, cudaEnableDefault, &q) == cudaSuccess && fn) {
            int fd = -1;
            if (reinterpret_cast<GetHandle>(fn)(&fd, reinterpret_cast<CUdeviceptr>(addr), length,
                                                CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD, 0) == CUDA_SUCCESS && fd >= 0) {
                mr = ibv_reg_dmabuf_mr(c_->pd, 0, length, reinterpret_cast<std::uint64_t>(addr), fd, access);
                ::close(fd);
            }
        }
#endif
        if (!mr) mr = ibv_reg_mr(c_->pd, addr, length, access);  // peer-memory kernel module
        if (!mr) throw std::runtime_error("rdma gdr: device memory registration unavailable (no dma-buf, no peer memory)");
        return MemoryRegion{addr, length, mr->lkey, mr->rkey, reinterpret_cast<std::uint64_t>(mr)};
    }

    void deregister(const MemoryRegion& mr) override {
        if (mr.handle) ibv_dereg_mr(reinterpret_cast<ibv_mr*>(mr.handle));
    }

    std::unique_ptr<CompletionQueue> create_cq(int depth) override {
        auto cq = std::unique_ptr<IbCq>(new IbCq());
        cq->cq = ibv_create_cq(c_->ctx, depth, nullptr, nullptr, 0);
        if (!cq->cq) throw std::runtime_error("rdma: ibv_create_cq failed");
        return cq;
    }

    std::unique_ptr<QueuePair> create_qp(CompletionQueue* cq, int max_send_wr, int max_recv_wr) override {
        auto qp = std::unique_ptr<IbQp>(new IbQp());
        qp->c = c_;
        ibv_qp_init_attr init{};
        init.send_cq = init.recv_cq = static_cast<IbCq*>(cq)->cq;  // one shared completion queue
        init.qp_type = IBV_QPT_RC;
        init.sq_sig_all = 0;
        init.cap.max_send_wr = max_send_wr;
        init.cap.max_recv_wr = max_recv_wr;
        init.cap.max_send_sge = init.cap.max_recv_sge = 1;
        init.cap.max_inline_data = kMaxInlineData;
        qp->qp = ibv_create_qp(c_->pd, &init);
        if (!qp->qp) throw std::runtime_error("rdma: ibv_create_qp failed");
        qp->psn = static_cast<std::uint32_t>(qp->qp->qp_num * 2654435761u) & 0xffffffu;
        return qp;
    }

private:
    std::shared_ptr<Context> c_;
};

}  // namespace

std::shared_ptr<VerbsBackend> create_ibverbs_backend() { return std::make_shared<IbVerbs>(); }

}  // namespace b200ccl::transport::rdma

#endif  // B200CCL_ENABLE_RDMA_VERBS
