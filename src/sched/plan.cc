#include "sched/plan.h"

#include "core/env.h"

#include <algorithm>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace b200ccl::sched {

namespace {
constexpr std::size_t kLlPlanMaxBytes = 128u << 10;  // capacity of the low-latency receive slots
}

Tuning default_tuning() {
    // Measured on 8x B200 (NVSwitch), float sum, CUDA-event timing, maximum over ranks
    // (tables under tuning/):
    //  * 8 ranks, device time from CUDA-graph replay: one-shot 9.7 us up to 8 KiB; the multimem kernel
    //    10.6-10.9 us flat up to 64 KiB and fastest from 16 KiB (10.8 vs 11.8 us one-shot) to 1 GiB
    //    (822 GB/s bus bandwidth); peer two-shot 10.4 us at 16-32 KiB and ahead of one-shot from there.
    //    64 CTAs beat 128 for multimem from 32 MiB up; two-shot likes 128 CTAs (199 vs 234 us at 64 MiB).
    //  * 4 ranks: one-shot 8.5 us up to 8 KiB, two-shot 9.3 us at 16-64 KiB, multimem fastest from
    //    128 KiB (10.3 vs 13.1 us) and level with two-shot at >= 4 MiB (608 vs 601 GB/s at 64 MiB).
    //  * 2 ranks: one-shot wins up to 1 MiB (15.7 us), two-shot above (585 GB/s at 64 MiB); multimem is
    //    slower than peer access there (366 GB/s) and is not used.
    Tuning t{};
    for (int n = 0; n <= kMaxRanks; ++n) t.oneshot_max_bytes[n] = 8u << 10;
    t.oneshot_max_bytes[1] = 0;
    t.oneshot_max_bytes[2] = 1u << 20;
    t.oneshot_max_bytes[3] = 16u << 10;
    t.nvls_min_bytes = 16u << 10;
    t.max_ctas = 128;
    //  * Multimem kernel, 8 ranks, unroll x CTAs: fewer loads in flight are faster. 64 MiB: 726 GB/s with 2 loads
    //    per thread on 48 CTAs, 722 (2, 64), 710 (4, 48), 692 (4, 64), 638 (8, 64), 587 (8, 128); 256 MiB: 818 (2, 48)
    //    down to 760 (8, 128).
    t.nvls_max_ctas = 48;
    t.nvls_staged_max_ctas = 64;
    t.nvls_unroll = 2;
    t.twoshot_max_ctas = 128;
    t.bytes_per_cta = 32u << 10;
    t.oneshot_bytes_per_cta = 8u << 10;
    //  * Low-latency kernel across NVLink, 2 ranks, graph replay: 3.4-3.6 us for 1-16 KiB and 4.2 us at 32 KiB
    //    against 7.5-10.7 us for one-shot (its two barrier round trips).
    //    8 ranks: 4.0-4.5 us up to 16 KiB, 5.6 us at 32 KiB, 7.3 us at 64 KiB against 11.2 us for the multimem
    //    kernel and 10.4-14 us for one-shot; at 128 KiB it falls behind (12.0 vs 11.5 us).
    //    4 ranks: 3.7-4.0 us up to 16 KiB, 6.6 us at 64 KiB (multimem 11.6), 9.7 us at 128 KiB (14.0);
    //    2 ranks: 3.3-3.5 us up to 16 KiB, 8.3 us at 128 KiB (two-shot 12.0).
    t.ll_max_bytes = 64u << 10;
    t.ll_max_bytes_upto4 = 128u << 10;
    //  * Tile pipeline for buffers peers cannot address against copy / barrier / reduce / barrier / copy:
    //    8 ranks 246 vs 224 us at 64 MiB, 835 vs 861 us at 256 MiB, 3142 vs 3414 us at 1 GiB; 2 ranks 152 vs 153 us
    //    at 64 MiB, 1711 vs 2271 us at 1 GiB.
    //    4 ranks (switch reduce stage): 214 vs 236 us at 64 MiB, 710 vs 929 us at 256 MiB, 2494-2610 vs 3704 us at 1 GiB;
    //    96 CTAs with one load in flight per thread: 479 / 568 / 646 GB/s at 64 MiB / 256 MiB / 1 GiB, 64 CTAs with two:
    //    471 / 567 / 617, 128 CTAs with two: 480 / 575 / 615 (per-tile times double with the CTA count: the switch is the limit).
    t.pipeline_min_bytes = 128u << 20;
    t.pipeline_min_bytes_upto4 = 64u << 20;
    t.pipeline_nvls_unroll = 1;
    t.pipeline_tile_bytes = 256u << 10;
    t.pipeline_max_ctas = 96;
    t.pipeline_peer_max_ctas = 128;
    return t;
}

Tuning tuning_from_text(const std::string& text, const Tuning& base, const std::string& origin) {
    Tuning t = base;
    std::istringstream in(text);
    std::string line;
    int lineno = 0;
    auto trim = [](std::string s) {
        const auto b = s.find_first_not_of(" \t\r");
        if (b == std::string::npos) return std::string();
        return s.substr(b, s.find_last_not_of(" \t\r") - b + 1);
    };
    while (std::getline(in, line)) {
        ++lineno;
        const auto hash = line.find('#');
        if (hash != std::string::npos) line.erase(hash);
        line = trim(line);
        if (line.empty()) continue;
        const std::string where = origin + ":" + std::to_string(lineno) + ": ";
        const auto eq = line.find('=');
        if (eq == std::string::npos) throw std::invalid_argument(where + "expected 'key = value'");
        const std::string key = trim(line.substr(0, eq)), value = trim(line.substr(eq + 1));
        std::size_t bytes = 0;
        if (!env::parse_bytes(value, &bytes)) throw std::invalid_argument(where + "bad value '" + value + "' for " + key);
        const int as_int = static_cast<int>(std::min<std::size_t>(bytes, 1u << 20));
        if (key == "oneshot_max_bytes") {
            for (int n = 2; n <= kMaxRanks; ++n) t.oneshot_max_bytes[n] = bytes;
        } else if (key.rfind("oneshot_max_bytes.", 0) == 0) {
            const std::string nstr = key.substr(18);
            char* end = nullptr;
            const long n = std::strtol(nstr.c_str(), &end, 10);
            if (nstr.empty() || *end != '\0' || n < 2 || n > kMaxRanks)
                throw std::invalid_argument(where + "rank count in '" + key + "' must be 2.." + std::to_string(kMaxRanks));
            t.oneshot_max_bytes[n] = bytes;
        } else if (key == "nvls_min_bytes") t.nvls_min_bytes = bytes;
        else if (key == "max_ctas") t.max_ctas = std::max(as_int, 1);
        else if (key == "nvls_max_ctas") t.nvls_max_ctas = t.nvls_staged_max_ctas = std::max(as_int, 1);
        else if (key == "nvls_staged_max_ctas") t.nvls_staged_max_ctas = std::max(as_int, 1);
        else if (key == "twoshot_max_ctas") t.twoshot_max_ctas = std::max(as_int, 1);
        else if (key == "nvls_unroll") t.nvls_unroll = as_int;
        else if (key == "bytes_per_cta") t.bytes_per_cta = std::max<std::size_t>(bytes, 1);
        else if (key == "oneshot_bytes_per_cta") t.oneshot_bytes_per_cta = std::max<std::size_t>(bytes, 1);
        else if (key == "ll_max_bytes") t.ll_max_bytes = t.ll_max_bytes_upto4 = std::min(bytes, kLlPlanMaxBytes);
        else if (key == "ll_max_bytes_upto4") t.ll_max_bytes_upto4 = std::min(bytes, kLlPlanMaxBytes);
        else if (key == "wide32") t.wide32 = bytes != 0;
        else if (key == "block_threads") {
            if (as_int < 32 || as_int > 512 || as_int % 32 != 0) throw std::invalid_argument(where + "block_threads must be a multiple of 32 between 32 and 512");
            t.block_threads = as_int;
        }
        else if (key == "pipeline_min_bytes") t.pipeline_min_bytes = t.pipeline_min_bytes_upto4 = bytes;
        else if (key == "pipeline_min_bytes_upto4") t.pipeline_min_bytes_upto4 = bytes;
        else if (key == "pipeline_nvls_unroll") t.pipeline_nvls_unroll = std::max(as_int, 1);
        else if (key == "pipeline_tile_bytes") t.pipeline_tile_bytes = std::max<std::size_t>(bytes / 4096 * 4096, 32u << 10);
        else if (key == "pipeline_max_ctas") t.pipeline_max_ctas = std::max(as_int, 1);
        else if (key == "pipeline_peer_max_ctas") t.pipeline_peer_max_ctas = std::max(as_int, 1);
        else throw std::invalid_argument(where + "unknown key '" + key + "'");
    }
    return t;
}

Tuning tuning_from_file(const std::string& path, const Tuning& base) {
    std::ifstream f(path);
    if (!f) throw std::invalid_argument("tuning file '" + path + "' cannot be read");
    std::stringstream text;
    text << f.rdbuf();
    return tuning_from_text(text.str(), base, path);
}

Tuning tuning_from_env() {
    Tuning t = default_tuning();
    if (const char* path = env::get("B200CCL_TUNING_FILE")) t = tuning_from_file(path, t);
    if (env::get("B200CCL_ONESHOT_MAX_BYTES")) {
        const std::size_t v = env::get_bytes("B200CCL_ONESHOT_MAX_BYTES", 0);
        for (int n = 0; n <= kMaxRanks; ++n) t.oneshot_max_bytes[n] = v;
    }
    t.nvls_min_bytes = env::get_bytes("B200CCL_NVLS_MIN_BYTES", t.nvls_min_bytes);
    if (env::get("B200CCL_MAX_CTAS")) {
        t.max_ctas = static_cast<int>(env::get_int("B200CCL_MAX_CTAS", t.max_ctas));
        t.nvls_max_ctas = t.nvls_staged_max_ctas = t.twoshot_max_ctas = t.max_ctas;  // an explicit cap applies to every algorithm
    }
    if (env::get("B200CCL_NVLS_MAX_CTAS"))
        t.nvls_max_ctas = t.nvls_staged_max_ctas = static_cast<int>(env::get_int("B200CCL_NVLS_MAX_CTAS", t.nvls_max_ctas));
    t.nvls_unroll = static_cast<int>(env::get_int("B200CCL_NVLS_UNROLL", t.nvls_unroll));
    t.bytes_per_cta = env::get_bytes("B200CCL_BYTES_PER_CTA", t.bytes_per_cta);
    t.oneshot_bytes_per_cta = env::get_bytes("B200CCL_ONESHOT_BYTES_PER_CTA", t.oneshot_bytes_per_cta);
    if (env::get("B200CCL_LL_MAX_BYTES"))
        t.ll_max_bytes = t.ll_max_bytes_upto4 = std::min<std::size_t>(env::get_bytes("B200CCL_LL_MAX_BYTES", 0), kLlPlanMaxBytes);
    t.wide32 = env::get_bool("B200CCL_WIDE32", t.wide32);
    t.block_threads = static_cast<int>(env::get_int("B200CCL_BLOCK_THREADS", t.block_threads, "NANO_NCCL_BLOCK_THREADS"));
    if (t.block_threads < 32 || t.block_threads > 512 || t.block_threads % 32 != 0)
        throw std::invalid_argument("B200CCL_BLOCK_THREADS must be a multiple of 32 between 32 and 512");
    if (env::get("B200CCL_PIPELINE_MIN_BYTES"))
        t.pipeline_min_bytes = t.pipeline_min_bytes_upto4 = env::get_bytes("B200CCL_PIPELINE_MIN_BYTES", 0);
    t.pipeline_nvls_unroll = std::max(1, static_cast<int>(env::get_int("B200CCL_PIPELINE_NVLS_UNROLL", t.pipeline_nvls_unroll)));
    t.pipeline_tile_bytes = std::max<std::size_t>(env::get_bytes("B200CCL_PIPELINE_TILE_BYTES", t.pipeline_tile_bytes) / 4096 * 4096, 32u << 10);
    t.pipeline_max_ctas = std::max(1, static_cast<int>(env::get_int("B200CCL_PIPELINE_MAX_CTAS", t.pipeline_max_ctas)));
    t.pipeline_peer_max_ctas = std::max(1, static_cast<int>(env::get_int("B200CCL_PIPELINE_PEER_MAX_CTAS", t.pipeline_peer_max_ctas)));
    return t;
}

std::size_t message_bytes(const CallShape& s) {
    const std::size_t one = s.count * dtype_size(s.dtype);
    return s.collective == Collective::AllReduce ? one : one * static_cast<std::size_t>(s.nranks);
}

namespace {

int grid_for(std::size_t bytes_this_rank_handles, const Tuning& t, int cap, std::size_t per_cta = 0) {
    const std::size_t per = std::max<std::size_t>(per_cta ? per_cta : t.bytes_per_cta, 1);
    std::size_t g = (bytes_this_rank_handles + per - 1) / per;
    g = std::max<std::size_t>(g, 1);
    return static_cast<int>(std::min<std::size_t>(g, static_cast<std::size_t>(std::max(cap, 1))));
}

bool nvls_usable(const CallShape& s) {
    // At two ranks the switch saves no traffic over direct peer access and measured slower.
    if (!s.wide || s.nranks < 3) return false;
    switch (s.collective) {
        case Collective::AllReduce: {
            // A side that peers cannot address is staged; the staging arena may itself be multicast-bound.
            const bool in_ok = s.input_multicast || (!s.peers_read_input && s.staging_multicast);
            const bool out_ok = s.output_multicast || (!s.peers_write_output && s.staging_multicast);
            return (s.redop == RedOp::Sum || s.redop == RedOp::Avg) && in_ok && out_ok;
        }
        case Collective::ReduceScatter:
            return (s.redop == RedOp::Sum || s.redop == RedOp::Avg) && s.input_multicast;
        case Collective::AllGather:
            return s.output_multicast;
    }
    return false;
}

}  // namespace

Plan make_plan(const CallShape& s, Algo forced, const Tuning& t) {
    Plan p;
    const int cap = std::max(1, std::min(s.max_ctas > 0 ? s.max_ctas : t.max_ctas, t.max_ctas));
    const std::size_t bytes = message_bytes(s);
    const std::size_t esz = dtype_size(s.dtype);

    if (s.ring_only || forced == Algo::Ring) {
        p.algo = Algo::Ring;
        p.grid = 0;  // the ring path sizes itself by channels
        return p;
    }
    if (s.nranks == 1) {
        // One rank: every collective is a copy of `count` elements. 16-byte aligned buffers go through
        // the TMA bulk-copy kernel (one CTA per SM, capped by max_ctas); anything else through the
        // element-wise path of the one-shot kernel, which degenerates to a local copy.
        p.algo = s.wide ? Algo::Copy : Algo::OneShot;
        p.grid = s.wide ? (cap < default_tuning().max_ctas ? cap : 148) : grid_for(bytes, t, 148);
        p.gather_mode = 1;
        return p;
    }

    const bool nvls_ok = nvls_usable(s);
    if (forced == Algo::Nvls && !nvls_ok) {
        p.error = "algo nvls needs symmetric (multicast-bound) buffers, 16-byte alignment and sum/avg";
        return p;
    }

    if (s.collective == Collective::AllGather) {
        if (forced == Algo::Nvls || (forced == Algo::Auto && nvls_ok && bytes >= t.nvls_min_bytes)) {
            p.algo = Algo::Nvls;
            p.gather_mode = 2;
        } else if (s.peers_write_output) {
            p.algo = Algo::OneShot;
            p.gather_mode = 0;
        } else {
            p.algo = Algo::OneShot;
            p.gather_mode = 1;
            p.stage_in = !s.peers_read_input;
        }
        p.grid = grid_for(s.count * esz * (p.gather_mode == 1 ? s.nranks : 1), t, cap);
        return p;
    }

    if (s.collective == Collective::ReduceScatter) {
        p.algo = (forced == Algo::Nvls || (forced == Algo::Auto && nvls_ok && bytes >= t.nvls_min_bytes))
                     ? Algo::Nvls : Algo::OneShot;
        p.stage_in = p.algo != Algo::Nvls && !s.peers_read_input;
        p.grid = grid_for(s.count * esz * (p.stage_in ? s.nranks : 1), t, cap);
        return p;
    }

    // AllReduce
    const bool ll_fits = s.word_aligned && bytes <= kLlPlanMaxBytes && s.nranks >= 2;
    if (forced == Algo::LowLatency && !ll_fits) {
        p.error = "algo ll takes 4-byte aligned all_reduce messages of at most 128 KiB";
        return p;
    }
    if (forced == Algo::LowLatency || (forced == Algo::Auto && ll_fits && bytes <= (s.nranks <= 4 ? t.ll_max_bytes_upto4 : t.ll_max_bytes))) {
        p.algo = Algo::LowLatency;  // neither buffer needs to be peer-addressable: no staging
        p.grid = 8;
        return p;
    }
    // Buffers that peers cannot address, large enough for the tile pipeline: both sides pass through
    // the staging arena (a side that peers could address is simply copied locally).
    const bool needs_staging = !s.peers_read_input || !s.peers_write_output;
    if (forced == Algo::Pipeline && !s.wide) {
        p.error = "algo pipeline needs 16-byte aligned buffers and a message that is a multiple of 16 bytes";
        return p;
    }
    if (forced == Algo::Pipeline || (forced == Algo::Auto && needs_staging && s.wide &&
                                     bytes >= (s.nranks <= 4 ? t.pipeline_min_bytes_upto4 : t.pipeline_min_bytes))) {
        p.algo = Algo::Pipeline;
        p.stage_in = p.stage_out = true;
        p.pipe_nvls = s.staging_multicast && s.nranks >= 3 && (s.redop == RedOp::Sum || s.redop == RedOp::Avg);
        // The peer-load reduce stage needs more CTAs than the switch one to keep NVLink busy.
        const int grid_max = std::max(1, std::min(cap, p.pipe_nvls ? t.pipeline_max_ctas : t.pipeline_peer_max_ctas));
        const std::size_t min_tile = 32u << 10;
        const std::size_t grid = std::max<std::size_t>(1, std::min<std::size_t>(static_cast<std::size_t>(grid_max), bytes / min_tile));
        const std::size_t per_cta = (bytes + grid - 1) / grid;
        // Every CTA gets the same number of tiles, each close to the preferred size.
        const std::size_t target = std::max<std::size_t>(t.pipeline_tile_bytes, min_tile);
        const std::size_t tiles_per_cta = std::max<std::size_t>(1, (per_cta + target / 2) / target);
        const std::size_t tile = ((per_cta + tiles_per_cta - 1) / tiles_per_cta + 4095) / 4096 * 4096;
        p.tile_bytes = tile;
        p.grid = static_cast<int>(std::min<std::size_t>(grid, (bytes + tile - 1) / tile));
        return p;
    }
    Algo algo = forced;
    if (algo == Algo::Auto) {
        if (nvls_ok && bytes >= t.nvls_min_bytes) algo = Algo::Nvls;
        else if (bytes <= t.oneshot_max_bytes[std::min(s.nranks, kMaxRanks)] && !s.in_place) algo = Algo::OneShot;
        else algo = Algo::TwoShot;
    }
    if (algo == Algo::OneShot && s.in_place && s.peers_read_input) {
        p.error = "one-shot all_reduce cannot run in place on buffers that peers read directly";
        return p;
    }
    p.algo = algo;
    if (algo == Algo::Nvls) {
        // Buffers that peers cannot address pass through the (multicast-bound) staging arena.
        p.stage_in = !s.peers_read_input;
        p.stage_out = !s.peers_write_output;
        // A staged call also copies the whole message in and out with these CTAs, which wants more of them than
        // the switch does (8 ranks, 64 MiB plain: 224 us on 64 CTAs, 236 us on 48).
        const bool staged = p.stage_in || p.stage_out;
        p.grid = grid_for(bytes / s.nranks * (staged ? s.nranks : 1), t,
                          std::min(cap, staged ? std::max(t.nvls_max_ctas, t.nvls_staged_max_ctas) : t.nvls_max_ctas));
    } else if (algo == Algo::OneShot) {
        p.stage_in = !s.peers_read_input;
        p.grid = grid_for(bytes, t, cap, t.oneshot_bytes_per_cta);
    } else {
        p.stage_in = !s.peers_read_input;
        p.stage_out = !s.peers_write_output;
        // Staging works on (input arena, output arena) pairs: if either side is staged the
        // kernel still reads/writes the other side in place.
        p.grid = grid_for(bytes / s.nranks * (p.stage_in || p.stage_out ? s.nranks : 1), t, std::min(cap, t.twoshot_max_ctas));
    }
    return p;
}

}  // namespace b200ccl::sched
