// Loopback "fabric" behind the stand-in verbs header of this folder. See infiniband/verbs.h here.
#include <infiniband/verbs.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <vector>

namespace {

struct Mr { char* addr; std::size_t length; };

struct PendingSend {
    ibv_send_wr wr;
    ibv_sge sge;
    std::vector<char> inline_copy;  // payload captured at post time for IBV_SEND_INLINE
};

struct RecvSlot { uint64_t wr_id; ibv_sge sge; };

struct Cq {
    ibv_cq pub;
    std::deque<ibv_wc> done;
    bool overrun = false;
};

struct Qp {
    ibv_qp pub;
    ibv_qp_cap cap{};
    uint32_t dest_qpn = 0, rq_psn = 0, sq_psn = 0;
    int path_mtu = 0;
    std::deque<PendingSend> sq;   // posted, not yet executed (in order)
    std::deque<RecvSlot> rq;
    unsigned unreaped = 0;        // send queue entries not yet released by a signalled completion
    bool error = false;
};

struct World {
    std::mutex mu;
    int device_count = 1;
    ibv_device device{};
    ibv_device* list[2] = {nullptr, nullptr};
    ibv_port_attr port{};
    std::map<uint32_t, Qp*> qps;
    std::map<uint32_t, Mr> mrs;  // by key (lkey == rkey here)
    uint32_t next_qpn = 0x100, next_key = 0x1000, next_handle = 1;
    fake_ibv_counters counters{};
    World() { reset_locked(); }
    void reset_locked() {
        device_count = 1;
        std::snprintf(device.name, sizeof(device.name), "fake0");
        std::memset(&port, 0, sizeof(port));
        port.state = IBV_PORT_ACTIVE;
        port.max_mtu = IBV_MTU_4096;
        port.active_mtu = IBV_MTU_4096;
        port.gid_tbl_len = 8;
        port.lid = 7;
        port.link_layer = IBV_LINK_LAYER_INFINIBAND;
        counters.sends = counters.signaled = counters.inline_sends = counters.rdma_writes = 0;
        counters.recvs = counters.rnr_waits = 0;
    }
};

World& world() {
    static World w;
    return w;
}

Cq* cq_of(ibv_cq* c) { return reinterpret_cast<Cq*>(c); }
Qp* qp_of(ibv_qp* q) { return reinterpret_cast<Qp*>(q); }

void complete(Cq* cq, const ibv_wc& wc) {
    if (static_cast<int>(cq->done.size()) >= cq->pub.cqe) {
        cq->overrun = true;
        return;
    }
    cq->done.push_back(wc);
}

bool covers(World& w, uint32_t key, uint64_t addr, uint32_t length) {
    auto it = w.mrs.find(key);
    if (it == w.mrs.end()) return false;
    const uint64_t base = reinterpret_cast<uint64_t>(it->second.addr);
    return addr >= base && addr + length <= base + it->second.length;
}

void fail_send(Qp* qp, const PendingSend& p, ibv_wc_status status) {
    ibv_wc wc{};
    wc.wr_id = p.wr.wr_id;
    wc.status = status;
    wc.opcode = IBV_WC_SEND;
    wc.qp_num = qp->pub.qp_num;
    complete(cq_of(qp->pub.send_cq), wc);
    qp->error = true;
    qp->pub.state = IBV_QPS_ERR;
}

// Executes as many queued sends of `qp` as the peer can take, in order.
void drain(World& w, Qp* qp) {
    while (!qp->sq.empty() && !qp->error) {
        auto peer_it = w.qps.find(qp->dest_qpn);
        if (peer_it == w.qps.end()) return;  // the peer does not exist (yet): stays queued, as a retry would
        Qp* peer = peer_it->second;
        if (peer->pub.state != IBV_QPS_RTR && peer->pub.state != IBV_QPS_RTS) return;
        PendingSend& p = qp->sq.front();
        const char* src = p.inline_copy.empty() ? reinterpret_cast<const char*>(p.sge.addr) : p.inline_copy.data();
        const uint32_t len = p.wr.num_sge ? p.sge.length : 0;
        const bool needs_recv = p.wr.opcode == IBV_WR_SEND || p.wr.opcode == IBV_WR_RDMA_WRITE_WITH_IMM;
        if (needs_recv && peer->rq.empty()) {
            ++w.counters.rnr_waits;  // receiver not ready: retried until a receive is posted (rnr_retry = 7)
            return;
        }
        if (peer->rq_psn != qp->sq_psn || peer->dest_qpn != qp->pub.qp_num) {
            fail_send(qp, p, IBV_WC_RETRY_EXC_ERR);  // the two ends were not wired to each other
            return;
        }
        ibv_wc rwc{};
        if (p.wr.opcode == IBV_WR_SEND) {
            RecvSlot slot = peer->rq.front();
            peer->rq.pop_front();
            rwc.wr_id = slot.wr_id;
            rwc.opcode = IBV_WC_RECV;
            rwc.qp_num = peer->pub.qp_num;
            rwc.src_qp = qp->pub.qp_num;
            if (len > slot.sge.length) {
                rwc.status = IBV_WC_LOC_LEN_ERR;
                complete(cq_of(peer->pub.recv_cq), rwc);
                fail_send(qp, p, IBV_WC_REM_INV_REQ_ERR);
                return;
            }
            if (len) std::memcpy(reinterpret_cast<char*>(slot.sge.addr), src, len);
            rwc.status = IBV_WC_SUCCESS;
            rwc.byte_len = len;
            complete(cq_of(peer->pub.recv_cq), rwc);
        } else {
            if (len && !covers(w, p.wr.wr.rdma.rkey, p.wr.wr.rdma.remote_addr, len)) {
                fail_send(qp, p, IBV_WC_REM_ACCESS_ERR);
                return;
            }
            if (len) std::memcpy(reinterpret_cast<char*>(p.wr.wr.rdma.remote_addr), src, len);
            ++w.counters.rdma_writes;
            if (p.wr.opcode == IBV_WR_RDMA_WRITE_WITH_IMM) {
                RecvSlot slot = peer->rq.front();
                peer->rq.pop_front();
                rwc.wr_id = slot.wr_id;
                rwc.opcode = IBV_WC_RECV_RDMA_WITH_IMM;
                rwc.status = IBV_WC_SUCCESS;
                rwc.byte_len = len;
                rwc.imm_data = p.wr.imm_data;
                rwc.wc_flags = IBV_WC_WITH_IMM;
                rwc.qp_num = peer->pub.qp_num;
                rwc.src_qp = qp->pub.qp_num;
                complete(cq_of(peer->pub.recv_cq), rwc);
            }
        }
        if (p.wr.send_flags & IBV_SEND_SIGNALED) {
            ibv_wc swc{};
            swc.wr_id = p.wr.wr_id;
            swc.status = IBV_WC_SUCCESS;
            swc.opcode = p.wr.opcode == IBV_WR_SEND ? IBV_WC_SEND : IBV_WC_RDMA_WRITE;
            swc.qp_num = qp->pub.qp_num;
            complete(cq_of(qp->pub.send_cq), swc);
            qp->unreaped = static_cast<unsigned>(qp->sq.size()) - 1;  // everything up to here is released
        }
        qp->sq.pop_front();
    }
}

}  // namespace

extern "C" {

ibv_device** ibv_get_device_list(int* num_devices) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    if (num_devices) *num_devices = w.device_count;
    if (w.device_count == 0) return nullptr;
    w.list[0] = &w.device;
    w.list[1] = nullptr;
    ++w.counters.live_objects;
    return w.list;
}
void ibv_free_device_list(ibv_device** list) {
    if (!list) return;
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    --w.counters.live_objects;
}
const char* ibv_get_device_name(ibv_device* device) { return device->name; }

ibv_context* ibv_open_device(ibv_device* device) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    ibv_context* c = new ibv_context{device, 1};
    ++w.counters.live_objects;
    return c;
}
int ibv_close_device(ibv_context* context) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    delete context;
    --w.counters.live_objects;
    return 0;
}
int ibv_query_port(ibv_context*, uint8_t port_num, ibv_port_attr* port_attr) {
    if (port_num != 1) return EINVAL;
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    *port_attr = w.port;
    return 0;
}
int ibv_query_gid(ibv_context*, uint8_t port_num, int index, ibv_gid* gid) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    if (port_num != 1 || index < 0 || index >= w.port.gid_tbl_len) return EINVAL;
    std::memset(gid, 0, sizeof(*gid));
    gid->raw[0] = 0xfe;
    gid->raw[1] = 0x80;
    gid->raw[15] = static_cast<uint8_t>(0x10 + index);
    return 0;
}
ibv_pd* ibv_alloc_pd(ibv_context* context) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    ++w.counters.live_objects;
    return new ibv_pd{context, w.next_handle++};
}
int ibv_dealloc_pd(ibv_pd* pd) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    delete pd;
    --w.counters.live_objects;
    return 0;
}
ibv_mr* ibv_reg_mr(ibv_pd* pd, void* addr, size_t length, int access) {
    if (!pd || !addr || length == 0 || !(access & IBV_ACCESS_LOCAL_WRITE)) {
        errno = EINVAL;
        return nullptr;
    }
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    const uint32_t key = w.next_key++;
    w.mrs[key] = Mr{static_cast<char*>(addr), length};
    ++w.counters.live_objects;
    return new ibv_mr{pd->context, pd, addr, length, w.next_handle++, key, key};
}
ibv_mr* ibv_reg_dmabuf_mr(ibv_pd*, uint64_t, size_t, uint64_t, int, int) {
    errno = EOPNOTSUPP;  // no dma-buf importer here
    return nullptr;
}
int ibv_dereg_mr(ibv_mr* mr) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    w.mrs.erase(mr->lkey);
    delete mr;
    --w.counters.live_objects;
    return 0;
}
ibv_cq* ibv_create_cq(ibv_context* context, int cqe, void* cq_context, void*, int) {
    if (cqe <= 0) {
        errno = EINVAL;
        return nullptr;
    }
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    Cq* cq = new Cq;
    cq->pub = ibv_cq{context, cq_context, w.next_handle++, cqe};
    ++w.counters.live_objects;
    return &cq->pub;
}
int ibv_destroy_cq(ibv_cq* cq) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    for (auto& kv : w.qps)
        if (kv.second->pub.send_cq == cq || kv.second->pub.recv_cq == cq) return EBUSY;  // queue pairs still use it
    delete cq_of(cq);
    --w.counters.live_objects;
    return 0;
}
ibv_qp* ibv_create_qp(ibv_pd* pd, ibv_qp_init_attr* init) {
    if (!pd || !init || !init->send_cq || !init->recv_cq || init->qp_type != IBV_QPT_RC || init->cap.max_send_sge < 1 ||
        init->cap.max_recv_sge < 1 || init->cap.max_send_wr == 0 || init->cap.max_inline_data > 256) {
        errno = EINVAL;
        return nullptr;
    }
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    Qp* qp = new Qp;
    std::memset(&qp->pub, 0, sizeof(qp->pub));
    qp->pub.context = pd->context;
    qp->pub.pd = pd;
    qp->pub.send_cq = init->send_cq;
    qp->pub.recv_cq = init->recv_cq;
    qp->pub.handle = w.next_handle++;
    qp->pub.qp_num = w.next_qpn++;
    qp->pub.state = IBV_QPS_RESET;
    qp->pub.qp_type = IBV_QPT_RC;
    qp->cap = init->cap;
    w.qps[qp->pub.qp_num] = qp;
    ++w.counters.live_objects;
    return &qp->pub;
}
int ibv_destroy_qp(ibv_qp* qp) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    w.qps.erase(qp->qp_num);
    delete qp_of(qp);
    --w.counters.live_objects;
    return 0;
}

int ibv_modify_qp(ibv_qp* q, ibv_qp_attr* a, int mask) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    Qp* qp = qp_of(q);
    if (!(mask & IBV_QP_STATE)) return EINVAL;
    const int init_mask = IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS;
    const int rtr_mask = IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN |
                         IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER;
    const int rts_mask = IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN |
                         IBV_QP_MAX_QP_RD_ATOMIC;
    switch (a->qp_state) {
        case IBV_QPS_INIT:
            if (q->state != IBV_QPS_RESET || (mask & init_mask) != init_mask || a->port_num != 1) return EINVAL;
            break;
        case IBV_QPS_RTR:
            if (q->state != IBV_QPS_INIT || (mask & rtr_mask) != rtr_mask) return EINVAL;
            if (a->path_mtu < IBV_MTU_256 || a->path_mtu > w.port.active_mtu || a->ah_attr.port_num != 1) return EINVAL;
            if (a->min_rnr_timer > 31 || a->rq_psn > 0xffffffu) return EINVAL;
            // RoCE (and a zero LID) cannot be addressed without a global route.
            if ((w.port.link_layer == IBV_LINK_LAYER_ETHERNET || a->ah_attr.dlid == 0) && !a->ah_attr.is_global) return EINVAL;
            if (a->ah_attr.is_global && a->ah_attr.grh.sgid_index >= w.port.gid_tbl_len) return EINVAL;
            qp->dest_qpn = a->dest_qp_num;
            qp->rq_psn = a->rq_psn;
            qp->path_mtu = a->path_mtu;
            break;
        case IBV_QPS_RTS:
            if (q->state != IBV_QPS_RTR || (mask & rts_mask) != rts_mask) return EINVAL;
            if (a->retry_cnt > 7 || a->rnr_retry > 7 || a->timeout > 31 || a->sq_psn > 0xffffffu) return EINVAL;
            qp->sq_psn = a->sq_psn;
            break;
        default:
            return EINVAL;
    }
    q->state = a->qp_state;
    // A peer may have queued sends before this end was ready to receive.
    for (auto& kv : w.qps)
        if (kv.second->dest_qpn == q->qp_num) drain(w, kv.second);
    return 0;
}

int ibv_post_send(ibv_qp* q, ibv_send_wr* wr, ibv_send_wr** bad_wr) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    Qp* qp = qp_of(q);
    for (; wr; wr = wr->next) {
        const uint32_t len = wr->num_sge ? wr->sg_list[0].length : 0;
        const bool inl = wr->send_flags & IBV_SEND_INLINE;
        int err = 0;
        if (q->state != IBV_QPS_RTS || wr->num_sge > 1) err = EINVAL;
        else if (qp->unreaped >= qp->cap.max_send_wr) err = ENOMEM;  // nothing signalled released the queue
        else if (inl && len > qp->cap.max_inline_data) err = EINVAL;
        else if (!inl && len && !covers(w, wr->sg_list[0].lkey, wr->sg_list[0].addr, len)) err = EINVAL;
        if (err) {
            if (bad_wr) *bad_wr = wr;
            return err;
        }
        PendingSend p;
        p.wr = *wr;
        p.wr.next = nullptr;
        p.sge = wr->num_sge ? wr->sg_list[0] : ibv_sge{};
        p.wr.sg_list = nullptr;
        if (inl && len) p.inline_copy.assign(reinterpret_cast<const char*>(p.sge.addr), reinterpret_cast<const char*>(p.sge.addr) + len);
        ++w.counters.sends;
        if (wr->send_flags & IBV_SEND_SIGNALED) ++w.counters.signaled;
        if (inl) ++w.counters.inline_sends;
        qp->sq.push_back(std::move(p));
        ++qp->unreaped;
    }
    drain(w, qp);
    return 0;
}

int ibv_post_recv(ibv_qp* q, ibv_recv_wr* wr, ibv_recv_wr** bad_wr) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    Qp* qp = qp_of(q);
    for (; wr; wr = wr->next) {
        int err = 0;
        if (q->state == IBV_QPS_RESET || wr->num_sge != 1) err = EINVAL;
        else if (qp->rq.size() >= qp->cap.max_recv_wr) err = ENOMEM;
        else if (wr->sg_list[0].length && !covers(w, wr->sg_list[0].lkey, wr->sg_list[0].addr, wr->sg_list[0].length)) err = EINVAL;
        if (err) {
            if (bad_wr) *bad_wr = wr;
            return err;
        }
        qp->rq.push_back(RecvSlot{wr->wr_id, wr->sg_list[0]});
        ++w.counters.recvs;
    }
    for (auto& kv : w.qps)
        if (kv.second->dest_qpn == q->qp_num) drain(w, kv.second);
    return 0;
}

int ibv_poll_cq(ibv_cq* c, int num_entries, ibv_wc* wc) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    Cq* cq = cq_of(c);
    if (cq->overrun) return -1;
    int n = 0;
    while (n < num_entries && !cq->done.empty()) {
        wc[n++] = cq->done.front();
        cq->done.pop_front();
    }
    return n;
}

void fake_ibv_reset(void) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    w.reset_locked();
}
void fake_ibv_set_device_count(int count) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    w.device_count = count;
}
void fake_ibv_set_port(enum ibv_port_state state, int link_layer, uint16_t lid, enum ibv_mtu active_mtu) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    w.port.state = state;
    w.port.link_layer = static_cast<uint8_t>(link_layer);
    w.port.lid = lid;
    w.port.active_mtu = active_mtu;
}
struct fake_ibv_counters fake_ibv_get_counters(void) {
    World& w = world();
    std::lock_guard<std::mutex> lock(w.mu);
    return w.counters;
}

}  // extern "C"
