// Argument and configuration contract, without a GPU. Key words follow the reference's API test
// (tests/public_api.cu:668-724): "one entry per rank", "non-null", "positive", "reduction",
// "in-place", "unsupported dtype", "visible sequence".
#include "check.h"
#include "b200ccl/communicator.h"
#include "b200ccl/types.h"
#include "collective/validate.h"
#include "core/env.h"
#include "sched/plan.h"
#include "sched/transport_plan.h"

#include <cstring>

using namespace b200ccl;

int main() {
    int a = 0, b = 0;
    CollectiveArgs ok;
    ok.send_buffers = {&a, &a};
    ok.recv_buffers = {&b, &b};
    ok.streams = {nullptr, nullptr};
    ok.count = 4;
    validate_collective_args(Collective::AllReduce, ok, 2, false);

    auto bad = ok;
    bad.streams.pop_back();
    t_expect_throw([&] { validate_collective_args(Collective::AllReduce, bad, 2, false); }, "one entry per rank", "sizes");
    bad = ok; bad.count = 0;
    t_expect_throw([&] { validate_collective_args(Collective::AllReduce, bad, 2, false); }, "positive", "count");
    bad = ok; bad.send_buffers[1] = nullptr;
    t_expect_throw([&] { validate_collective_args(Collective::AllReduce, bad, 2, false); }, "non-null", "null");
    bad = ok; bad.redop = static_cast<RedOp>(9);
    t_expect_throw([&] { validate_collective_args(Collective::AllReduce, bad, 2, false); }, "reduction", "redop");
    bad = ok; bad.dtype = static_cast<DType>(7);
    t_expect_throw([&] { validate_collective_args(Collective::AllReduce, bad, 2, false); }, "unsupported dtype", "dtype");
    bad = ok; bad.recv_buffers[0] = &a;
    t_expect_throw([&] { validate_collective_args(Collective::AllReduce, bad, 2, false); }, "in-place", "in-place");
    validate_collective_args(Collective::AllReduce, bad, 2, true);  // explicitly allowed
    t_expect_throw([&] { validate_collective_args(Collective::ReduceScatter, bad, 2, true); }, "in-place", "rs in-place");
    t_expect_throw([&] { validate_collective_args(Collective::AllGather, bad, 2, true); }, "all_gather", "names the collective");

    CommunicatorConfig cfg;
    t_expect_throw([&] { validate_config(cfg, 4); }, "at least one device", "empty devices");
    cfg.devices = {0, 5};
    t_expect_throw([&] { validate_config(cfg, 4); }, "visible sequence", "device range");
    cfg.devices = {1, 1};
    t_expect_throw([&] { validate_config(cfg, 4); }, "twice", "duplicate");
    cfg.devices = {0, 1, 2};
    validate_config(cfg, 4);
    cfg.max_ctas = -1;
    t_expect_throw([&] { validate_config(cfg, 4); }, "max_ctas", "negative CTA cap");
    cfg.max_ctas = 16;
    validate_config(cfg, 4);
    cfg.transport = TransportKind::Mixed;
    t_expect_throw([&] { validate_config(cfg, 4); }, "mixed", "mixed cannot be requested");
    cfg = CommunicatorConfig{};
    cfg.devices = {0, 1};
    cfg.loopback = true;
    t_expect_throw([&] { validate_config(cfg, 4); }, "exactly one device", "loopback devices");

    // names and parsers
    DType d; RedOp r; TransportKind t; Algo al; Collective c;
    T_CHECK(parse_dtype("bf16", &d) && d == DType::BFloat16 && !parse_dtype("int8", &d));
    T_CHECK(parse_redop("avg", &r) && r == RedOp::Avg && !parse_redop("prod", &r));
    T_CHECK(parse_transport("p2p", &t) && t == TransportKind::P2p);
    T_CHECK(!parse_transport("socket", &t) && !parse_transport("mixed", &t));  // reported, never requested
    T_CHECK(std::strcmp(transport_name(TransportKind::Socket), "socket") == 0);
    T_CHECK(parse_algo("ring_simple", &al) && al == Algo::Ring && parse_algo("nvls", &al));
    T_CHECK(parse_collective("reduce_scatter", &c) && c == Collective::ReduceScatter);
    T_CHECK(dtype_size(DType::Float) == 4 && dtype_size(DType::BFloat16) == 2);
    T_CHECK(dtype_default_epsilon(DType::Float16) == 1e-2f);
    const auto sizes = make_sizes(262144, 67108864, 4);
    T_CHECK(sizes.size() == 5 && sizes.front() == 262144 && sizes.back() == 67108864);
    T_CHECK(all_reduce_busbw_gbs(100.0, 4) == 150.0 && busbw_gbs(Collective::AllGather, 100.0, 4) == 75.0);

    // environment parsing is strict
    bool flag = false; std::size_t bytes = 0;
    T_CHECK(env::parse_bool("On", &flag) && flag && env::parse_bool("0", &flag) && !flag && !env::parse_bool("yes", &flag));
    T_CHECK(env::parse_bytes("32M", &bytes) && bytes == (32u << 20) && env::parse_bytes("1G", &bytes) && !env::parse_bytes("x", &bytes));

    // planner
    sched::CallShape s;
    s.nranks = 8; s.count = 1 << 10; s.wide = true; s.peers_read_input = s.peers_write_output = true;
    auto plan = sched::make_plan(s, Algo::Auto, sched::default_tuning());
    T_CHECK(plan.algo == Algo::OneShot && !plan.stage_in);
    s.count = 16 << 20;
    plan = sched::make_plan(s, Algo::Auto, sched::default_tuning());
    T_CHECK(plan.algo == Algo::TwoShot && plan.grid > 1);
    s.input_multicast = s.output_multicast = true;
    plan = sched::make_plan(s, Algo::Auto, sched::default_tuning());
    T_CHECK(plan.algo == Algo::Nvls);
    s.redop = RedOp::Max;  // the switch cannot be trusted to propagate NaN → peer kernels
    plan = sched::make_plan(s, Algo::Auto, sched::default_tuning());
    T_CHECK(plan.algo == Algo::TwoShot);
    T_CHECK(!sched::make_plan(s, Algo::Nvls, sched::default_tuning()).error.empty());
    s = sched::CallShape{}; s.nranks = 4; s.count = 64 << 20; s.wide = true;  // plain buffers of another process, 256 MiB
    plan = sched::make_plan(s, Algo::Auto, sched::default_tuning());
    T_CHECK(plan.stage_in && plan.stage_out && plan.algo == Algo::Pipeline);  // large: the tile pipeline
    T_CHECK(plan.tile_bytes >= (32u << 10) && plan.tile_bytes % 4096 == 0 && plan.grid >= 1 && plan.grid <= 128);
    T_CHECK((static_cast<std::size_t>(256) << 20) / plan.tile_bytes >= static_cast<std::size_t>(plan.grid));  // no CTA without a tile
    {   // every CTA gets the same number of tiles
        const std::size_t tiles = ((static_cast<std::size_t>(256) << 20) + plan.tile_bytes - 1) / plan.tile_bytes;
        T_CHECK(tiles % static_cast<std::size_t>(plan.grid) == 0 || tiles / plan.grid >= 1);
    }
    T_CHECK(!plan.pipe_nvls);                      // the arena has no multicast alias in this shape
    s.staging_multicast = true;
    T_CHECK(sched::make_plan(s, Algo::Auto, sched::default_tuning()).pipe_nvls);
    s.redop = RedOp::Min;                          // max/min never go through the switch
    T_CHECK(!sched::make_plan(s, Algo::Auto, sched::default_tuning()).pipe_nvls);
    s.redop = RedOp::Sum;
    s.count = 1 << 20;                             // 4 MiB: below the pipeline threshold → copy, barrier, reduce, barrier, copy
    plan = sched::make_plan(s, Algo::Auto, sched::default_tuning());
    T_CHECK(plan.stage_in && plan.stage_out && plan.algo != Algo::Pipeline);
    T_CHECK(sched::make_plan(s, Algo::Pipeline, sched::default_tuning()).algo == Algo::Pipeline);  // on request at any size
    s.wide = false;
    T_CHECK(!sched::make_plan(s, Algo::Pipeline, sched::default_tuning()).error.empty());
    s.wide = true;
    s.ring_only = true;
    T_CHECK(sched::make_plan(s, Algo::Auto, sched::default_tuning()).algo == Algo::Ring);
    // process layouts and per-edge transport plans (synthetic 2x2 topologies, as the reference's
    // tests/public_api.cu --topology mode and tests/p2p_topology.cu do)
    sched::ProcessLayout two_by_two;
    two_by_two.nranks = 4;
    two_by_two.first_rank = {0, 2};
    two_by_two.rank_count = {2, 2};
    two_by_two.validate();
    T_CHECK(two_by_two.distributed() && two_by_two.owner_of(1) == 0 && two_by_two.owner_of(2) == 1 && two_by_two.owner_of(9) == -1);
    auto tp = sched::make_ring_transport_plan(two_by_two, TransportKind::P2p, TransportKind::Socket, false);
    T_CHECK(tp.edge_kinds.size() == 4);
    T_CHECK(tp.edge_kinds[0] == TransportKind::P2p && tp.edge_kinds[1] == TransportKind::Socket);   // 1->2 crosses
    T_CHECK(tp.edge_kinds[2] == TransportKind::P2p && tp.edge_kinds[3] == TransportKind::Socket);   // 3->0 crosses
    T_CHECK(tp.resolved_kind() == TransportKind::Mixed);
    T_CHECK(tp.describe().find("edge 1->2: socket") != std::string::npos && tp.describe().find("edge 3->0: socket") != std::string::npos);
    tp = sched::make_ring_transport_plan(two_by_two, TransportKind::P2p, TransportKind::P2p, false);
    T_CHECK(tp.resolved_kind() == TransportKind::P2p);
    tp = sched::make_ring_transport_plan(two_by_two, TransportKind::Shm, TransportKind::Rdma, false);
    T_CHECK(tp.resolved_kind() == TransportKind::Mixed && tp.edge_kinds[0] == TransportKind::Shm && tp.edge_kinds[1] == TransportKind::Rdma);
    sched::ProcessLayout one;
    one.nranks = 4; one.first_rank = {0}; one.rank_count = {4};
    T_CHECK(!one.distributed());
    T_CHECK(sched::make_ring_transport_plan(one, TransportKind::Shm, TransportKind::P2p, false).resolved_kind() == TransportKind::Shm);
    T_CHECK(sched::make_ring_transport_plan(one, TransportKind::P2p, TransportKind::Rdma, true).resolved_kind() == TransportKind::Rdma);
    sched::ProcessLayout four_by_one;
    four_by_one.nranks = 4; four_by_one.first_rank = {0, 1, 2, 3}; four_by_one.rank_count = {1, 1, 1, 1};
    T_CHECK(sched::make_ring_transport_plan(four_by_one, TransportKind::P2p, TransportKind::Socket, false).resolved_kind() == TransportKind::Socket);
    sched::ProcessLayout solo;
    solo.nranks = 1; solo.first_rank = {0}; solo.rank_count = {1};
    T_CHECK(sched::make_ring_transport_plan(solo, TransportKind::P2p, TransportKind::P2p, false).resolved_kind(TransportKind::P2p) == TransportKind::P2p);
    sched::ProcessLayout gap = two_by_two;
    gap.first_rank = {0, 3};
    t_expect_throw([&] { gap.validate(); }, "do not follow", "gap in ranks");
    gap = two_by_two; gap.nranks = 5;
    t_expect_throw([&] { gap.validate(); }, "own 4 ranks", "sum mismatch");
    t_expect_throw([&] { sched::make_ring_transport_plan(two_by_two, TransportKind::Socket, TransportKind::P2p, false); }, "inside a process", "local kind");
    t_expect_throw([&] { sched::make_ring_transport_plan(two_by_two, TransportKind::P2p, TransportKind::Shm, false); }, "between processes", "cross kind");
    std::puts("validate ok");
    return 0;
}
