// Attention entry points of the C ABI: argument rules, work planning, dispatch.
//
// Stands in for MetalExecutor::runPagedFlashAttention / encodePagedFlashAttention
// (compiler/runtime/metal_runtime.mm:7727-7826, 7074-7166). The reference copies
// its four u32 host arrays to the device on every call and gives one threadgroup
// to each (request, head) (mm:7101-7107, 7155). Here the host arrays are turned
// into a work plan - per-CTA tile lists balanced over the whole GPU - which is
// uploaded once and reused for as long as the caller keeps passing the same
// tables (the reference's walker passes identical tables for each of its 22
// layers, compiler/runtime/batched_walker.cpp:316-325).
#include "attn_internal.hpp"
#include "qkv_rope.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <queue>

namespace mlcb {

static constexpr size_t kMaxPassLayersApi = 64;   // layers of one whole-pass launch (decode_pass_supported checks it)

struct PlanKey {
    size_t batch = 0, H = 0, KVH = 0, D = 0, P = 0, capacity = 0, n_flat = 0;
    int causal = 0;
    bool operator==(const PlanKey& o) const {
        return batch == o.batch && H == o.H && KVH == o.KVH && D == o.D && P == o.P &&
               capacity == o.capacity && n_flat == o.n_flat && causal == o.causal;
    }
};

}  // namespace mlcb

// A device-resident work plan for one set of page tables. Created explicitly by
// mlc_attn_plan_create, or implicitly (and cached) by the entry points that take
// host arrays.
struct mlc_attn_plan {
    mlcb::PlanKey key;
    std::vector<uint32_t> tables;  // pt_flat | pt_off | seq_lens | q_pos as passed by the caller
    uint8_t* host = nullptr;       // pinned image of the device blob
    uint8_t* dev = nullptr;
    size_t cap = 0;
    cudaEvent_t uploaded = nullptr;
    // Bookkeeping of the launches that read the device copy (mutable: a plan is const to the entry points that
    // use it): the stream epoch of the last such launch, and whether the last upload went to the copy stream
    // and the next launch therefore has to wait for it.
    mutable uint64_t use_epoch = 0;
    mutable bool upload_on_copy_stream = false;
    mlcb::DecodePlanView view;
    mlcb::DecodePlanView view_pass;   // work lists of the whole-pass launch (pass_ready says whether they exist)
    const uint32_t* d_page_ids = nullptr;  // this step's (page, slot) per request, when given
    const uint32_t* d_slots = nullptr;
    uint64_t stamp = 0;
};

namespace mlcb {

struct AttnPlanCache {
    static constexpr int kEntries = 4;
    mlc_attn_plan e[kEntries];
    uint64_t clock = 0;
};

static void release_plan_buffers(mlc_attn_plan& p) {
    if (p.uploaded) cudaEventSynchronize(p.uploaded);   // an upload may still be under way on the copy stream
    if (p.host) cudaFreeHost(p.host);
    if (p.dev) cudaFree(p.dev);
    if (p.uploaded) cudaEventDestroy(p.uploaded);
    p.host = p.dev = nullptr;
    p.uploaded = nullptr;
    p.cap = 0;
}

// Called by every entry point that launches with a plan: the launch must see the plan's latest upload (which
// may have gone to the copy stream), and the plan remembers in which stream epoch it was last used.
int use_plan(mlc_ctx* ctx, const mlc_attn_plan* plan) {
    if (plan->upload_on_copy_stream) {
        // inside a capture the event counts as an external one (a wait node that is long satisfied at replay)
        MLCB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, plan->uploaded, ctx->capturing ? cudaEventWaitExternal : 0));
        plan->upload_on_copy_stream = false;
    }
    // a launch captured into a graph can be replayed at any time: such a plan is only ever updated in stream order
    plan->use_epoch = ctx->capturing ? UINT64_MAX : std::max(plan->use_epoch, ctx->sync_epoch);
    return MLC_OK;
}

void destroy_plan_cache(mlc_ctx* ctx) {
    if (!ctx->plan_cache) return;
    for (auto& p : ctx->plan_cache->e) release_plan_buffers(p);
    delete ctx->plan_cache;
    ctx->plan_cache = nullptr;
}

namespace {

int env_int(const char* name, int dflt) {
    const char* v = std::getenv(name);
    return v && *v ? std::atoi(v) : dflt;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Builds the plan image for one set of tables into `p` and uploads it.
// Lists of varying length for consecutive slices in two flat arrays (a vector per slice costs an
// allocation or several each, ~100 us for the 1024 slices of a unit-mode plan). Lists are appended
// to in non-decreasing slice order.
template <typename T>
struct FlatLists {
    std::vector<uint32_t> off;  // off[i] = start of list i; off[n] = total once finished
    std::vector<T> items;
    uint32_t cur = 0, n = 0;
    void reset(uint32_t count, size_t expect) {
        n = count;
        off.assign(static_cast<size_t>(count) + 1, 0);
        items.clear();
        items.reserve(expect);
        cur = 0;
    }
    void push(uint32_t list, const T& v) {
        while (cur < list) off[++cur] = static_cast<uint32_t>(items.size());
        items.push_back(v);
    }
    uint32_t size_so_far(uint32_t list) {  // list >= cur
        while (cur < list) off[++cur] = static_cast<uint32_t>(items.size());
        return static_cast<uint32_t>(items.size()) - off[list];
    }
    void finish() {
        while (cur < n) off[++cur] = static_cast<uint32_t>(items.size());
    }
    uint32_t size(uint32_t list) const { return off[list + 1] - off[list]; }
    T& at(uint32_t list, uint32_t i) { return items[off[list] + i]; }
    const T* data(uint32_t list) const { return items.data() + off[list]; }
};

int build_plan(mlc_ctx* ctx, mlc_attn_plan& p, const uint32_t* pt_flat, const uint32_t* pt_off,
               const uint32_t* seq_lens, const uint32_t* q_pos, const uint32_t* page_ids,
               const uint32_t* slots) {
    if (ctx->capturing)
        return ctx->fail(MLC_ERR_UNSUPPORTED, "new page tables inside a graph capture: create the plan before capturing");
    const PlanKey& k = p.key;
    const size_t N = k.batch;
    std::vector<uint32_t> eff(N), zero_rows;
    for (size_t r = 0; r < N; ++r) {
        uint32_t S = seq_lens[r];
        // kv_pos > q_pos masked (mm:2286): only [0, min(S, q_pos+1)) can contribute.
        if (k.causal && static_cast<uint64_t>(q_pos[r]) + 1 < S) S = q_pos[r] + 1;
        eff[r] = S;
        if (S == 0) zero_rows.push_back(static_cast<uint32_t>(r));
    }

    FlatLists<PieceDesc> cta_pieces;   // per plan slice, filled slice after slice
    FlatLists<uint32_t> cta_tiles;
    uint32_t n_cta = 0, max_pieces = 1, max_tiles = 1, n_slots = 0, n_segs = 0, n_unit_cuts = 0, stages = 3;
    // A decode step can fuse the row write into attention when the newest token of every
    // request (position seq_len - 1, where page_ids / slots must point) is attended to.
    bool fusable = page_ids != nullptr;
    for (size_t r = 0; r < N && fusable; ++r) {
        const uint32_t S = seq_lens[r];
        fusable = S > 0 && eff[r] == S && page_ids[r] == pt_flat[pt_off[r] + (S - 1) / k.P] &&
                  slots[r] == (S - 1) % k.P;
    }
    const bool tma = decode_tma_shape_supported(k.H, k.KVH, k.D, k.P, k.capacity);
    std::vector<SegDesc> segs;
    bool unit_mode = false;
    uint32_t unit_mode_hpc = 1;
    // second work list for whole-pass launches (see below); absent when the TMA kernel or the fused row write do not apply
    FlatLists<PieceDesc> pass_pieces;
    FlatLists<uint32_t> pass_tiles;
    bool pass_built = false, pass_same_as_primary = false;
    uint32_t pass_hpc = 1, pass_n_cta = 0, pass_max_pieces = 1, pass_max_tiles = 1, pass_stages = 1;
    uint32_t n_slices = 0;  // plan slices: one per CTA, or one per warp in unit mode
    if (tma) {
        // ---- which decomposition? -----------------------------------------------------------
        // split: requests cut over all CTAs along the sequence, 4 KV heads per CTA, split requests merged
        //        by a second kernel chained behind (on the critical path, longer with more parts);
        // unit : a (request, KV head) never leaves its CTA - longest-first packing of whole units onto
        //        the CTAs, the CTA's warps share a unit and merge in shared memory, no merge kernel; a
        //        unit that dwarfs a CTA's fair share is cut into runs on different CTAs (see below).
        // The estimate below is in microseconds and in "head tiles" (32 tokens of one head, K and V);
        // its constants come from timing both forms on B200 over a dozen batch shapes (per layer, in a
        // CUDA graph): ~0.18 us per head tile and SM when the HBM is shared by all SMs, ~0.135 us per
        // head tile (0.095 with 8 warps at head_dim 64) for the CTA that holds the longest unit, fixed costs of ~3 us (unit) and ~9 us plus
        // ~0.9 us per 12 parts of the most split request (split).
        const uint32_t TOKu = kTileTokens;
        const uint32_t UW = static_cast<uint32_t>(unit_warps(k.D));
        // Heads per CTA item (hpc): 1 = a unit is a (request, KV head) shared by all warps of a CTA; h > 1 = a
        // unit is a (request, group of h adjacent KV heads), warp w taking head w % h and part w / h of the
        // tiles, so that the CTA reads h adjacent 128-byte (256-byte at head_dim 128) chunks of every token
        // row together. Needs h | KVH and h | warps.
        // A launch per layer uses hpc = 1 (many small units balance a single layer best); the whole-pass
        // launch, which balances across layers, uses the largest h (measured on B200, 22 layers of 32
        // requests: 0.78 of the copy bandwidth with h = 1, 0.86 with 2, 0.88 with 4).
        const uint32_t hpc = 1;   // the per-layer kernel
        using UnitList = std::vector<std::pair<uint32_t, uint32_t>>;  // (tiles of a head x h, request * (KVH / h) + head group)
        uint64_t head_tiles = 0;
        for (size_t r = 0; r < N; ++r) head_tiles += static_cast<uint64_t>((eff[r] + TOKu - 1) / TOKu) * k.KVH;
        auto make_units = [&](uint32_t h) {
            UnitList u;
            const uint32_t groups = static_cast<uint32_t>(k.KVH) / h;
            for (size_t r = 0; r < N; ++r) {
                const uint32_t t = (eff[r] + TOKu - 1) / TOKu;
                if (!t) continue;
                for (uint32_t hg = 0; hg < groups; ++hg) u.emplace_back(t * h, static_cast<uint32_t>(r * groups + hg));
            }
            // (tiles, id) descending so that equal packings come out the same from call to call
            std::sort(u.begin(), u.end(), [](const auto& x, const auto& y) { return x.first != y.first ? x.first > y.first : x.second < y.second; });
            return u;
        };
        UnitList units = make_units(hpc);
        const int per_sm_u = std::max(env_int("MLC_B200_DECODE_CTAS_PER_SM", 1), 1);
        const uint32_t cta_cap = static_cast<uint32_t>(ctx->sm_count) * per_sm_u;
        // An item is a unit or, when cutting helps, a run of a unit's tiles: a unit much longer than a
        // CTA's fair share (all tiles / CTAs) is cut into equal runs that go to different CTAs; each
        // leaves a partial in the workspace and the CTA that brings a unit's last part combines them
        // (an arrival counter per cut unit, nobody waits). Items are packed by estimated time, longest
        // first onto the least loaded CTA: c_lone per tile, ~1 us per item (Q fetch, in-CTA exchange: a
        // CTA's items do not overlap), and for a run of a cut unit ~0.75 us + 0.135 us per part (store of
        // the partial, counter round trip, the last arrival's loads). Cutting pays when one unit dwarfs
        // a CTA's fair share (a lone 16384-token request: 47 -> 10 us per layer; 4 x 32768: 92 -> 27) and
        // costs when the batch is balanced already (cfg2 forced to cut at the fair share: 8.8 -> 13.6),
        // so a few run lengths are packed and the whole-unit packing stays unless a cut one is
        // estimated at least 10 % faster.
        struct Item { uint32_t tiles, id, lo, hi, part, n_parts, cut, cost_ns; };   // cut: index among the cut units
        struct Packing {
            std::vector<Item> items;
            std::vector<std::vector<uint32_t>> cta_items;   // indices into items
            uint64_t critical = 0;   // estimated time of the fullest CTA, ns
            uint32_t n_cta = 0, n_cut = 0, n_parts_total = 0;
        };
        const double f_dim = static_cast<double>(k.D) / 64.0;
        const double c_lone = k.D == 64 ? 0.095 : 0.135;  // us per head tile on the fullest CTA (8 warps at 64, 4 at 128)
        auto pack = [&](const UnitList& ulist, uint32_t cap_tiles, Packing& pk) {
            pk.items.clear();
            pk.n_cut = pk.n_parts_total = 0;
            for (const auto& u : ulist) {
                uint32_t parts = 1;
                if (cap_tiles && u.first > cap_tiles + cap_tiles / 4) parts = std::min<uint32_t>((u.first + cap_tiles - 1) / cap_tiles, 64u);
                for (uint32_t q = 0; q < parts; ++q) {
                    const uint32_t lo = static_cast<uint32_t>(static_cast<uint64_t>(u.first) * q / parts);
                    const uint32_t hi = static_cast<uint32_t>(static_cast<uint64_t>(u.first) * (q + 1) / parts);
                    const double us = f_dim * c_lone * (hi - lo) + 1.0 + (parts > 1 ? 0.75 + 0.135 * parts : 0.0);
                    pk.items.push_back(Item{hi - lo, u.second, lo, hi, q, parts, parts > 1 ? pk.n_cut : 0u,
                                            static_cast<uint32_t>(us * 1000.0)});
                }
                if (parts > 1) {
                    ++pk.n_cut;
                    pk.n_parts_total += parts;
                }
            }
            std::vector<uint32_t> order(pk.items.size());
            for (uint32_t i = 0; i < order.size(); ++i) order[i] = i;
            std::sort(order.begin(), order.end(), [&](uint32_t x, uint32_t y) {
                return pk.items[x].cost_ns != pk.items[y].cost_ns ? pk.items[x].cost_ns > pk.items[y].cost_ns : x < y;
            });
            pk.n_cta = static_cast<uint32_t>(std::min<size_t>(cta_cap, pk.items.size()));
            pk.cta_items.assign(pk.n_cta, {});
            pk.critical = 0;
            std::vector<std::pair<uint64_t, uint32_t>> heap;  // (load, cta), min-heap
            for (uint32_t c = 0; c < pk.n_cta; ++c) heap.emplace_back(0, c);
            auto cmp = [](const auto& x, const auto& y) { return x.first != y.first ? x.first > y.first : x.second > y.second; };
            std::make_heap(heap.begin(), heap.end(), cmp);
            for (uint32_t i : order) {
                std::pop_heap(heap.begin(), heap.end(), cmp);
                auto& slot = heap.back();
                pk.cta_items[slot.second].push_back(i);
                slot.first += pk.items[i].cost_ns;
                pk.critical = std::max(pk.critical, slot.first);
                std::push_heap(heap.begin(), heap.end(), cmp);
            }
        };
        Packing whole, cut, trial;
        Packing* chosen = nullptr;
        double t_unit = 0.0;
        if (!units.empty() && k.KVH <= kTileHbMask + 1) {
            const double f = f_dim;
            const double per_sm_tiles = static_cast<double>(head_tiles) / ctx->sm_count;
            const double t_stream = f * 0.18 * per_sm_tiles;   // all SMs sharing the HBM
            pack(units, 0, whole);
            chosen = &whole;
            t_unit = std::max(whole.critical * 1e-3, t_stream) + 2.0;
            // MLC_B200_DECODE_UNIT_CUT: 0 = never cut, otherwise the run lengths tried are this percentage
            // of 2.5x, 1.5x and 1x the fair share; MLC_B200_DECODE_UNIT_CUT_FORCE=1 cuts at that percentage.
            const int cut_pct = hpc > 1 ? 0 : env_int("MLC_B200_DECODE_UNIT_CUT", 100);   // head groups are never cut
            const bool force_cut = env_int("MLC_B200_DECODE_UNIT_CUT_FORCE", 0) != 0;
            const uint32_t fair = static_cast<uint32_t>((head_tiles + cta_cap - 1) / cta_cap);
            if (cut_pct > 0 && (force_cut || whole.critical * 1e-3 > 1.3 * t_stream)) {
                double best = force_cut ? 1e30 : t_unit * 0.9;
                uint32_t last_cap = 0;
                for (const int mult : {250, 150, 100}) {   // longest runs first: on a tie the fewer parts win
                    if (force_cut && mult != 100) continue;
                    const uint32_t cap_tiles = std::max<uint32_t>(static_cast<uint32_t>(static_cast<uint64_t>(fair) * cut_pct / 100 * mult / 100), 2 * UW);
                    if (cap_tiles == last_cap || units.front().first <= cap_tiles + cap_tiles / 4) continue;
                    last_cap = cap_tiles;
                    pack(units, cap_tiles, trial);
                    const double t_cut = std::max(trial.critical * 1e-3, t_stream) + 2.0;
                    if (trial.n_cut && t_cut < best) {
                        best = t_cut;
                        std::swap(cut, trial);
                        chosen = &cut;
                        t_unit = t_cut;
                    }
                }
            }
            const uint32_t n_hb_e = static_cast<uint32_t>((k.KVH + kDecodeWarps - 1) / kDecodeWarps);
            const double hb_tiles = static_cast<double>(head_tiles) / k.KVH * n_hb_e;      // tiles of the split form
            const double per_cta = std::max(1.0, hb_tiles / cta_cap);
            const double max_parts = std::min<double>(cta_cap, units.front().first / per_cta + 1.0);
            const double t_split = f * 0.185 * per_sm_tiles + 9.0 + 0.9 * std::ceil(max_parts / 12.0);
            const int forced = env_int("MLC_B200_DECODE_MODE", 0);  // 0 auto, 1 split, 2 unit
            unit_mode = forced == 2 || (forced == 0 && t_unit < t_split);
        }
        stages = static_cast<uint32_t>(std::min<int>(decode_tma_max_stages(k.H, k.KVH, k.D),
                                                     std::max(1, env_int("MLC_B200_DECODE_STAGES", k.D == 128 ? 2 : 3))));
        // Lays a packing out as per-warp piece and tile lists: slice rank * UW + w belongs to warp w of the CTA
        // with the rank-th largest load (the heaviest start first, and a whole-pass launch deals (layer,
        // rank) items to the SMs by this rank, see decode_body).
        auto emit_units = [&](const Packing& pk, uint32_t h, FlatLists<PieceDesc>& pieces, FlatLists<uint32_t>& tiles) {
            const uint32_t groups = static_cast<uint32_t>(k.KVH) / h;
            const uint32_t slices = pk.n_cta * UW;
            std::vector<uint32_t> cut_first_slot(pk.n_cut + 1, 0);
            for (const Item& it : pk.items)
                if (it.n_parts > 1 && it.part == 0) cut_first_slot[it.cut + 1] = it.n_parts;
            for (uint32_t i = 0; i < pk.n_cut; ++i) cut_first_slot[i + 1] += cut_first_slot[i];
            pieces.reset(slices, pk.items.size() * UW);
            tiles.reset(slices, static_cast<size_t>(head_tiles) + slices);
            std::vector<uint32_t> cta_rank(pk.n_cta);
            std::vector<uint64_t> cta_load(pk.n_cta, 0);
            for (uint32_t c = 0; c < pk.n_cta; ++c) {
                cta_rank[c] = c;
                for (uint32_t ii : pk.cta_items[c]) cta_load[c] += pk.items[ii].cost_ns;
            }
            std::stable_sort(cta_rank.begin(), cta_rank.end(), [&](uint32_t x, uint32_t y) { return cta_load[x] > cta_load[y]; });
            for (uint32_t rank = 0; rank < pk.n_cta; ++rank) {
                const uint32_t c = cta_rank[rank];
                for (uint32_t w = 0; w < UW; ++w) {
                    const uint32_t slice = rank * UW + w;
                    for (uint32_t ii : pk.cta_items[c]) {
                        const Item& it = pk.items[ii];
                        const size_t r = it.id / groups;
                        const uint32_t hd = static_cast<uint32_t>(it.id % groups) * h + w % h;   // this warp's KV head
                        const uint32_t T = (eff[r] + TOKu - 1) / TOKu;       // tiles of one head of the unit
                        // the warps of a head (all, or every h-th) share its run of tiles in equal parts
                        const uint32_t run = (it.hi - it.lo) / h, run_lo = it.lo / h, wparts = UW / h, wp = w / h;
                        const uint32_t share = (run + wparts - 1) / wparts;
                        const uint32_t lo = run_lo + std::min(wp * share, run), hi = run_lo + std::min((wp + 1) * share, run);
                        PieceDesc d{};
                        d.req = static_cast<uint32_t>(r);
                        d.hb = static_cast<uint16_t>(hd);   // the KV head itself
                        d.tile_begin = lo;
                        d.n_tiles = hi - lo;
                        d.n_parts = static_cast<uint16_t>(it.n_parts);
                        if (it.n_parts > 1) {
                            d.seg = it.cut;
                            d.seg_first_slot = cut_first_slot[it.cut];
                            d.part_slot = cut_first_slot[it.cut] + it.part;
                        }
                        const bool has_last = hi == T && hi > lo;
                        d.last_valid = static_cast<uint16_t>(has_last ? eff[r] - (T - 1) * TOKu : TOKu);
                        d.flags = (fusable && has_last) ? 1u : 0u;
                        pieces.push(slice, d);
                        for (uint32_t t = lo; t < hi; ++t) {
                            const uint64_t tok0 = static_cast<uint64_t>(t) * TOKu;
                            const uint32_t page = pt_flat[pt_off[r] + tok0 / k.P];
                            const uint32_t sub = static_cast<uint32_t>((tok0 % k.P) / TOKu);
                            const uint32_t fresh = (fusable && t + 1 == T) ? kTileFreshBit : 0u;
                            tiles.push(slice, page | (sub << kTileSubShift) | (hd << kTileHbShift) | fresh);
                        }
                    }
                }
            }
            pieces.finish();
            tiles.finish();
        };
        // the exchange area of the in-CTA merge must fit beside the rings
        uint32_t unit_stages = stages;
        while (unit_stages > 1 && decode_tma_smem_bytes(k.D, k.H / k.KVH > 8, unit_stages, true) > 227 * 1024 - 1024) --unit_stages;  // 1 KiB for the barriers
        pass_stages = unit_stages;
        if (unit_mode) {
            stages = unit_stages;
            unit_mode_hpc = hpc;
            const Packing& pk = *chosen;
            n_cta = pk.n_cta;
            n_slices = n_cta * UW;
            n_unit_cuts = pk.n_cut;
            n_slots = (pk.n_parts_total + kDecodeWarps - 1) / kDecodeWarps;   // the workspace is sized in groups of kDecodeWarps parts
            emit_units(pk, hpc, cta_pieces, cta_tiles);
        }
        // ---- the view a whole-pass launch uses: whole units of as many adjacent heads as the warps allow
        if (fusable && chosen && k.KVH <= kTileHbMask + 1 && env_int("MLC_B200_DECODE_PASS", 1) != 0) {
            uint32_t h = 1;
            for (uint32_t c = static_cast<uint32_t>(std::min<size_t>(k.KVH, UW)); c > 1; --c)
                if (k.KVH % c == 0 && UW % c == 0) { h = c; break; }
            if (const int forced_h = env_int("MLC_B200_DECODE_PASS_HPC", 0); forced_h > 0 && k.KVH % forced_h == 0 && UW % forced_h == 0)
                h = static_cast<uint32_t>(forced_h);
            pass_hpc = h;
            if (unit_mode && n_unit_cuts == 0 && h == hpc) {
                pass_same_as_primary = true;
            } else {
                const UnitList pass_units = make_units(h);
                Packing pass_pk;
                pack(pass_units, 0, pass_pk);
                pass_n_cta = pass_pk.n_cta;
                emit_units(pass_pk, h, pass_pieces, pass_tiles);
            }
            pass_built = true;
        }
    }
    if (tma && !unit_mode) {
        const uint32_t TOK = kTileTokens;
        const uint32_t n_hb = static_cast<uint32_t>((k.KVH + kDecodeWarps - 1) / kDecodeWarps);
        uint64_t total = 0;
        for (size_t r = 0; r < N; ++r) total += static_cast<uint64_t>((eff[r] + TOK - 1) / TOK) * n_hb;
        // One CTA per SM and ~100 KiB of ring per CTA where possible: a decode-step kernel
        // and its programmatic successor can then share an SM.
        int per_sm = env_int("MLC_B200_DECODE_CTAS_PER_SM", 1);
        uint64_t max_cta = static_cast<uint64_t>(ctx->sm_count) * std::max(per_sm, 1);
        int min_tiles = std::max(env_int("MLC_B200_DECODE_MIN_TILES", 1), 1);
        n_cta = static_cast<uint32_t>(std::max<uint64_t>(1, std::min<uint64_t>(max_cta, total / min_tiles)));
        n_slices = n_cta;
        cta_pieces.reset(n_cta, N * n_hb + n_cta);
        cta_tiles.reset(n_cta, total);
        uint32_t c = 0;
        uint64_t g = 0;  // global tile index
        auto cta_end = [&](uint32_t cc) { return (static_cast<uint64_t>(cc) + 1) * total / n_cta; };
        for (size_t r = 0; r < N; ++r) {
            const uint32_t tiles_r = (eff[r] + TOK - 1) / TOK;
            if (tiles_r == 0) continue;
            for (uint32_t hb = 0; hb < n_hb; ++hb) {
                uint32_t t = 0;
                std::vector<std::pair<uint32_t, uint32_t>> seg_pieces;  // (cta, index)
                while (t < tiles_r) {
                    while (g >= cta_end(c)) ++c;
                    uint32_t take = static_cast<uint32_t>(std::min<uint64_t>(tiles_r - t, cta_end(c) - g));
                    PieceDesc d{};
                    d.req = static_cast<uint32_t>(r);
                    d.hb = static_cast<uint16_t>(hb);
                    d.tile_begin = t;
                    d.n_tiles = take;
                    d.last_valid = static_cast<uint16_t>(
                        (t + take == tiles_r) ? eff[r] - (tiles_r - 1) * TOK : TOK);
                    d.flags = (fusable && t + take == tiles_r) ? 1u : 0u;
                    seg_pieces.emplace_back(c, cta_pieces.size_so_far(c));
                    cta_pieces.push(c, d);
                    for (uint32_t i = 0; i < take; ++i) {
                        uint64_t tok0 = static_cast<uint64_t>(t + i) * TOK;
                        uint32_t page = pt_flat[pt_off[r] + tok0 / k.P];
                        uint32_t sub = static_cast<uint32_t>((tok0 % k.P) / TOK);
                        uint32_t fresh = (fusable && t + i + 1 == tiles_r) ? kTileFreshBit : 0u;
                        cta_tiles.push(c, page | (sub << kTileSubShift) | (hb << kTileHbShift) | fresh);
                    }
                    t += take;
                    g += take;
                }
                uint16_t parts = static_cast<uint16_t>(seg_pieces.size());
                uint32_t first_slot = n_slots;
                for (size_t i = 0; i < seg_pieces.size(); ++i) {
                    PieceDesc& d = cta_pieces.at(seg_pieces[i].first, seg_pieces[i].second);
                    d.n_parts = parts;
                    d.seg = parts > 1 ? n_segs : 0;
                    d.seg_first_slot = first_slot;
                    d.part_slot = first_slot + static_cast<uint32_t>(i);
                }
                if (parts > 1) {
                    segs.push_back({static_cast<uint32_t>(r), hb, first_slot, parts});
                    n_slots += parts;
                    ++n_segs;
                }
            }
        }
    }
    if (n_slices) {
        cta_pieces.finish();
        cta_tiles.finish();
    }
    for (uint32_t i = 0; i < n_slices; ++i) {
        max_pieces = std::max<uint32_t>(max_pieces, cta_pieces.size(i));
        max_tiles = std::max<uint32_t>(max_tiles, cta_tiles.size(i));
    }
    const bool pass_own = pass_built && !pass_same_as_primary;   // the pass view has lists of its own
    const uint32_t pass_slices = pass_own ? pass_n_cta * static_cast<uint32_t>(unit_warps(k.D)) : 0;
    for (uint32_t i = 0; i < pass_slices; ++i) {
        pass_max_pieces = std::max<uint32_t>(pass_max_pieces, pass_pieces.size(i));
        pass_max_tiles = std::max<uint32_t>(pass_max_tiles, pass_tiles.size(i));
    }

    // ---- lay the image out
    size_t off = 0;
    const size_t off_counts = off;   off = align_up(off + size_t(n_slices) * 8, 16);
    // +512 / +256 bytes: the kernel reads 16 descriptors and 64 tile words per plan slice unconditionally
    const size_t off_pieces = off;   off = align_up(off + size_t(n_slices) * max_pieces * sizeof(PieceDesc) + 512, 16);
    const size_t off_tiles = off;    off = align_up(off + size_t(n_slices) * max_tiles * 4 + 256, 16);
    const size_t off_flat = off;     off = align_up(off + k.n_flat * 4, 16);
    const size_t off_ptoff = off;    off = align_up(off + (N + 1) * 4, 16);
    const size_t off_eff = off;      off = align_up(off + N * 4, 16);
    const size_t off_zero = off;     off = align_up(off + zero_rows.size() * 4, 16);
    const size_t off_segs = off;     off = align_up(off + segs.size() * sizeof(SegDesc), 16);
    const size_t off_ids = off;      off = align_up(off + (page_ids ? N * 4 : 0), 16);
    const size_t off_slots = off;    off = align_up(off + (slots ? N * 4 : 0), 16);
    const size_t off_pcounts = off;  off = align_up(off + size_t(pass_slices) * 8, 16);
    const size_t off_ppieces = off;  off = align_up(off + (pass_own ? size_t(pass_slices) * pass_max_pieces * sizeof(PieceDesc) + 512 : 0), 16);
    const size_t off_ptiles = off;   off = align_up(off + (pass_own ? size_t(pass_slices) * pass_max_tiles * 4 + 256 : 0), 16);
    const size_t bytes = std::max<size_t>(off, 16);

    if (p.uploaded) MLCB_CUDA(ctx, cudaEventSynchronize(p.uploaded));
    if (bytes > p.cap) {
        MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (p.host) cudaFreeHost(p.host);
        if (p.dev) cudaFree(p.dev);
        p.host = p.dev = nullptr;
        p.cap = 0;
        size_t want = align_up(bytes * 2, 4096);
        if (cudaHostAlloc(reinterpret_cast<void**>(&p.host), want, cudaHostAllocDefault) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void**>(&p.dev), want) != cudaSuccess)
            return ctx->fail(MLC_ERR_OOM, "plan buffer of %zu bytes unavailable", want);
        p.cap = want;
        ctx->allocations += 2;
    }
    if (!p.uploaded) MLCB_CUDA(ctx, cudaEventCreateWithFlags(&p.uploaded, cudaEventDisableTiming));

    std::memset(p.host, 0, bytes);
    auto* counts_h = reinterpret_cast<uint32_t*>(p.host + off_counts);
    auto* pieces_h = reinterpret_cast<PieceDesc*>(p.host + off_pieces);
    auto* tiles_h = reinterpret_cast<uint32_t*>(p.host + off_tiles);
    for (uint32_t i = 0; i < n_slices; ++i) {
        counts_h[2 * i] = cta_pieces.size(i);
        counts_h[2 * i + 1] = cta_tiles.size(i);
        std::copy(cta_pieces.data(i), cta_pieces.data(i) + cta_pieces.size(i), pieces_h + size_t(i) * max_pieces);
        std::copy(cta_tiles.data(i), cta_tiles.data(i) + cta_tiles.size(i), tiles_h + size_t(i) * max_tiles);
    }
    if (pass_own) {
        auto* pc = reinterpret_cast<uint32_t*>(p.host + off_pcounts);
        auto* pp = reinterpret_cast<PieceDesc*>(p.host + off_ppieces);
        auto* pt = reinterpret_cast<uint32_t*>(p.host + off_ptiles);
        for (uint32_t i = 0; i < pass_slices; ++i) {
            pc[2 * i] = pass_pieces.size(i);
            pc[2 * i + 1] = pass_tiles.size(i);
            std::copy(pass_pieces.data(i), pass_pieces.data(i) + pass_pieces.size(i), pp + size_t(i) * pass_max_pieces);
            std::copy(pass_tiles.data(i), pass_tiles.data(i) + pass_tiles.size(i), pt + size_t(i) * pass_max_tiles);
        }
    }
    if (k.n_flat) std::memcpy(p.host + off_flat, pt_flat, k.n_flat * 4);
    std::memcpy(p.host + off_ptoff, pt_off, (N + 1) * 4);
    std::memcpy(p.host + off_eff, eff.data(), N * 4);
    if (!zero_rows.empty()) std::memcpy(p.host + off_zero, zero_rows.data(), zero_rows.size() * 4);
    if (!segs.empty()) std::memcpy(p.host + off_segs, segs.data(), segs.size() * sizeof(SegDesc));
    if (page_ids) std::memcpy(p.host + off_ids, page_ids, N * 4);
    if (slots) std::memcpy(p.host + off_slots, slots, N * 4);
    // Where the upload goes: if the stream has been synchronised since the plan's last launch, nothing in flight
    // reads its device copy, and the upload runs on the copy stream beside whatever the main stream is doing
    // (the kernels of the pass that uses the OTHER plan, in a walker that alternates two). Otherwise in stream
    // order, behind the kernels already enqueued with the old tables.
    if (p.use_epoch < ctx->sync_epoch && !ctx->capturing) {
        if (!ctx->h2d_stream) MLCB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
        MLCB_CUDA(ctx, cudaMemcpyAsync(p.dev, p.host, bytes, cudaMemcpyHostToDevice, ctx->h2d_stream));
        MLCB_CUDA(ctx, cudaEventRecord(p.uploaded, ctx->h2d_stream));
        p.upload_on_copy_stream = true;
    } else {
        MLCB_CUDA(ctx, cudaMemcpyAsync(p.dev, p.host, bytes, cudaMemcpyHostToDevice, ctx->stream));
        MLCB_CUDA(ctx, cudaEventRecord(p.uploaded, ctx->stream));
        p.upload_on_copy_stream = false;
    }

    DecodePlanView& v = p.view;
    v.cta_counts = reinterpret_cast<const uint32_t*>(p.dev + off_counts);
    v.pieces = reinterpret_cast<const PieceDesc*>(p.dev + off_pieces);
    v.tile_pages = reinterpret_cast<const uint32_t*>(p.dev + off_tiles);
    v.pt_flat = reinterpret_cast<const uint32_t*>(p.dev + off_flat);
    v.pt_off = reinterpret_cast<const uint32_t*>(p.dev + off_ptoff);
    v.eff_len = reinterpret_cast<const uint32_t*>(p.dev + off_eff);
    v.zero_rows = reinterpret_cast<const uint32_t*>(p.dev + off_zero);
    v.seg_desc = reinterpret_cast<const SegDesc*>(p.dev + off_segs);
    v.has_tma = tma;
    v.step_fusable = tma && fusable;
    v.unit_mode = unit_mode;
    v.stages = stages;
    v.n_cta = n_cta;
    v.max_pieces = max_pieces;
    v.max_tiles = max_tiles;
    v.n_zero = static_cast<uint32_t>(zero_rows.size());
    v.n_slots = n_slots;
    v.n_segs = n_segs;
    v.n_unit_cuts = n_unit_cuts;
    v.hpc = unit_mode_hpc;
    // the view of whole-pass launches: the same lists when they already are whole units of the widest head
    // group, else the second set
    DecodePlanView& pv = p.view_pass;
    pv = v;
    pv.pass_ready = pass_built;
    if (pass_own) {
        pv.cta_counts = reinterpret_cast<const uint32_t*>(p.dev + off_pcounts);
        pv.pieces = reinterpret_cast<const PieceDesc*>(p.dev + off_ppieces);
        pv.tile_pages = reinterpret_cast<const uint32_t*>(p.dev + off_ptiles);
        pv.unit_mode = true;
        pv.stages = pass_stages;
        pv.n_cta = pass_n_cta;
        pv.max_pieces = pass_max_pieces;
        pv.max_tiles = pass_max_tiles;
        pv.n_slots = pv.n_segs = pv.n_unit_cuts = 0;
        pv.hpc = pass_hpc;
    }
    p.d_page_ids = page_ids ? reinterpret_cast<const uint32_t*>(p.dev + off_ids) : nullptr;
    p.d_slots = slots ? reinterpret_cast<const uint32_t*>(p.dev + off_slots) : nullptr;
    return MLC_OK;
}

// Argument rules shared by every entry point that takes the host tables.
int validate_tables(mlc_ctx* ctx, PlanKey& key, const void* k_pages, const uint32_t* pt_flat, size_t n_flat,
                    const uint32_t* pt_off, const uint32_t* seq_lens, const uint32_t* q_pos,
                    size_t capacity_pages) {
    // metal_runtime.mm:7742-7750
    if (key.batch == 0 || key.H == 0 || key.D == 0 || key.P == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (key.KVH == 0 || key.H % key.KVH != 0) return ctx->fail(MLC_ERR_INVALID_ARG, "num_heads must be a multiple of kv_heads");
    if (!pt_off || !seq_lens || !q_pos || (!pt_flat && n_flat)) return ctx->fail(MLC_ERR_INVALID_ARG, "null table");
    if (n_flat < pt_off[key.batch]) return ctx->fail(MLC_ERR_INVALID_ARG, "page_tables_flat shorter than the last offset");
    if (key.D > 256) return ctx->fail(MLC_ERR_UNSUPPORTED, "head_dim > 256");
    if (key.batch * key.H >= (size_t(1) << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch * heads too large");
    // checks the reference does not make
    key.capacity = resolve_capacity(ctx, k_pages, capacity_pages, key.P * key.KVH * key.D * 2);
    key.n_flat = pt_off[key.batch];
    for (size_t r = 0; r < key.batch; ++r) {
        if (pt_off[r + 1] < pt_off[r]) return ctx->fail(MLC_ERR_BOUNDS, "page_table_offsets not monotone at %zu", r);
        uint64_t room = static_cast<uint64_t>(pt_off[r + 1] - pt_off[r]) * key.P;
        if (seq_lens[r] > room)
            return ctx->fail(MLC_ERR_BOUNDS, "seq_lens[%zu]=%u exceeds its %u pages", r, seq_lens[r], pt_off[r + 1] - pt_off[r]);
    }
    if (key.capacity)
        for (size_t i = 0; i < key.n_flat; ++i)
            if (pt_flat[i] >= key.capacity)
                return ctx->fail(MLC_ERR_BOUNDS, "page_tables_flat[%zu]=%u >= capacity %zu", i, pt_flat[i], key.capacity);
    return MLC_OK;
}

int get_cached_plan(mlc_ctx* ctx, const PlanKey& key, const uint32_t* pt_flat, const uint32_t* pt_off,
                    const uint32_t* seq_lens, const uint32_t* q_pos, mlc_attn_plan** out) {
    if (!ctx->plan_cache) ctx->plan_cache = new AttnPlanCache();
    AttnPlanCache& pc = *ctx->plan_cache;
    const size_t N = key.batch;
    const size_t words = key.n_flat + (N + 1) + N + N;
    mlc_attn_plan* victim = &pc.e[0];
    for (auto& p : pc.e) {
        if (p.stamp && p.key == key && p.tables.size() == words) {
            const uint32_t* t = p.tables.data();
            if ((key.n_flat == 0 || !std::memcmp(t, pt_flat, key.n_flat * 4)) &&
                !std::memcmp(t + key.n_flat, pt_off, (N + 1) * 4) &&
                !std::memcmp(t + key.n_flat + N + 1, seq_lens, N * 4) &&
                !std::memcmp(t + key.n_flat + 2 * N + 1, q_pos, N * 4)) {
                p.stamp = ++pc.clock;
                *out = &p;
                return MLC_OK;
            }
        }
        if (p.stamp < victim->stamp) victim = &p;
    }
    mlc_attn_plan& p = *victim;
    p.key = key;
    p.tables.resize(words);
    if (key.n_flat) std::memcpy(p.tables.data(), pt_flat, key.n_flat * 4);
    std::memcpy(p.tables.data() + key.n_flat, pt_off, (N + 1) * 4);
    std::memcpy(p.tables.data() + key.n_flat + N + 1, seq_lens, N * 4);
    std::memcpy(p.tables.data() + key.n_flat + 2 * N + 1, q_pos, N * 4);
    p.stamp = 0;
    int st = build_plan(ctx, p, pt_flat, pt_off, seq_lens, q_pos, nullptr, nullptr);
    if (st != MLC_OK) return st;
    p.stamp = ++pc.clock;
    *out = &p;
    return MLC_OK;
}

int finish_sync(mlc_ctx* ctx, const char* what) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return ctx->fail(MLC_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
    uint32_t word = 0;
    MLCB_CUDA(ctx, cudaMemcpy(&word, ctx->d_err, 4, cudaMemcpyDeviceToHost));
    if (word) {
        reset_after_device_error(ctx);
        return ctx->fail(MLC_ERR_DEVICE_FLAG, "%s recorded error word 0x%x", what, word);
    }
    return MLC_OK;
}

// Launches attention for a validated call through `plan`.
int launch_with_plan(mlc_ctx* ctx, AttnArgs a, const mlc_attn_plan& plan) {
    const PlanKey& k = plan.key;
    if (!a.q || !a.k_pages || !a.v_pages || (!a.o && !a.o_partial)) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if ((a.q_dtype != MLC_F32 && a.q_dtype != MLC_F16) || (a.o_dtype != MLC_F32 && a.o_dtype != MLC_F16))
        return ctx->fail(MLC_ERR_INVALID_ARG, "dtype must be MLC_F32 or MLC_F16");
    if (a.o_partial && !a.ml_partial) return ctx->fail(MLC_ERR_INVALID_ARG, "partial output needs both buffers");
    a.batch = k.batch; a.H = k.H; a.KVH = k.KVH; a.D = k.D; a.P = k.P; a.capacity = k.capacity;
    if (a.scale <= 0.f) a.scale = 1.0f / std::sqrt(static_cast<float>(a.D));  // mm:7133
    if (plan.view.has_tma && !ctx->force_general && decode_tma_pointers_supported(a)) {
        ctx->last_attention_kernel = 2;
        return launch_attention_decode_tma(ctx, a, plan.view);
    }
    ctx->last_attention_kernel = 1;
    return launch_attention_general(ctx, a, plan.view.pt_flat, plan.view.pt_off, plan.view.eff_len);
}

int attention_impl(mlc_ctx* ctx, bool sync, AttnArgs a, const uint32_t* pt_flat, size_t n_flat,
                   const uint32_t* pt_off, const uint32_t* seq_lens, const uint32_t* q_pos,
                   int causal, size_t capacity_pages) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!a.q || !a.k_pages || !a.v_pages || (!a.o && !a.o_partial)) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    PlanKey key;
    key.batch = a.batch; key.H = a.H; key.KVH = a.KVH; key.D = a.D; key.P = a.P; key.causal = causal ? 1 : 0;
    int st = validate_tables(ctx, key, a.k_pages, pt_flat, n_flat, pt_off, seq_lens, q_pos, capacity_pages);
    if (st != MLC_OK) return st;
    if (!sync && !ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    DeviceGuard guard(ctx->device);
    mlc_attn_plan* plan = nullptr;
    if ((st = get_cached_plan(ctx, key, pt_flat, pt_off, seq_lens, q_pos, &plan)) != MLC_OK) return st;
    if ((st = use_plan(ctx, plan)) != MLC_OK) return st;
    if ((st = launch_with_plan(ctx, a, *plan)) != MLC_OK) return st;
    return sync ? finish_sync(ctx, "attention") : MLC_OK;
}

}  // namespace

int launch_attention_with_plan(mlc_ctx* ctx, AttnArgs a, const mlc_attn_plan* plan) {
    return launch_with_plan(ctx, a, *plan);
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

int mlc_run_paged_flash_attention(mlc_ctx* ctx, const void* q, const void* k_pages,
                                  const void* v_pages, void* o, const uint32_t* page_tables_flat,
                                  size_t n_page_tables_flat, const uint32_t* page_table_offsets,
                                  const uint32_t* seq_lens, const uint32_t* q_positions,
                                  size_t batch, size_t num_heads, size_t kv_heads, size_t head_dim,
                                  size_t page_size_tokens, int apply_causal, float scale,
                                  int q_dtype, int o_dtype, size_t capacity_pages) {
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
    a.batch = batch; a.H = num_heads; a.KVH = kv_heads; a.D = head_dim; a.P = page_size_tokens;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    return attention_impl(ctx, true, a, page_tables_flat, n_page_tables_flat, page_table_offsets,
                          seq_lens, q_positions, apply_causal, capacity_pages);
}

int mlc_encode_paged_flash_attention(mlc_ctx* ctx, const void* q, const void* k_pages,
                                     const void* v_pages, void* o,
                                     const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                     const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                     const uint32_t* q_positions, size_t batch, size_t num_heads,
                                     size_t kv_heads, size_t head_dim, size_t page_size_tokens,
                                     int apply_causal, float scale, int q_dtype, int o_dtype,
                                     size_t capacity_pages) {
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
    a.batch = batch; a.H = num_heads; a.KVH = kv_heads; a.D = head_dim; a.P = page_size_tokens;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    return attention_impl(ctx, false, a, page_tables_flat, n_page_tables_flat, page_table_offsets,
                          seq_lens, q_positions, apply_causal, capacity_pages);
}

int mlc_ctx_last_attention_kernel(const mlc_ctx* ctx) { return ctx ? ctx->last_attention_kernel : 0; }

int mlc_attn_plan_create(mlc_ctx* ctx, const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                         const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                         const uint32_t* q_positions, const uint32_t* page_ids,
                         const uint32_t* slots_in_page, size_t batch, size_t num_heads,
                         size_t kv_heads, size_t head_dim, size_t page_size_tokens, int apply_causal,
                         size_t capacity_pages, mlc_attn_plan** out) {
    if (!ctx || !out) return MLC_ERR_INVALID_ARG;
    *out = nullptr;
    if ((page_ids == nullptr) != (slots_in_page == nullptr)) return ctx->fail(MLC_ERR_INVALID_ARG, "page_ids and slots_in_page go together");
    PlanKey key;
    key.batch = batch; key.H = num_heads; key.KVH = kv_heads; key.D = head_dim; key.P = page_size_tokens;
    key.causal = apply_causal ? 1 : 0;
    int st = validate_tables(ctx, key, nullptr, page_tables_flat, n_page_tables_flat, page_table_offsets,
                             seq_lens, q_positions, capacity_pages);
    if (st != MLC_OK) return st;
    if (page_ids)
        for (size_t r = 0; r < batch; ++r) {
            if (key.capacity && page_ids[r] >= key.capacity)
                return ctx->fail(MLC_ERR_BOUNDS, "page_ids[%zu]=%u >= capacity %zu", r, page_ids[r], key.capacity);
            if (slots_in_page[r] >= page_size_tokens)
                return ctx->fail(MLC_ERR_BOUNDS, "slots_in_page[%zu]=%u >= page size", r, slots_in_page[r]);
        }
    DeviceGuard guard(ctx->device);
    auto* p = new mlc_attn_plan();
    p->key = key;
    st = build_plan(ctx, *p, page_tables_flat, page_table_offsets, seq_lens, q_positions, page_ids, slots_in_page);
    if (st != MLC_OK) {
        release_plan_buffers(*p);
        delete p;
        return st;
    }
    *out = p;
    return MLC_OK;
}

int mlc_attn_plan_update(mlc_ctx* ctx, mlc_attn_plan* plan, const uint32_t* page_tables_flat,
                         size_t n_page_tables_flat, const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                         const uint32_t* q_positions, const uint32_t* page_ids, const uint32_t* slots_in_page,
                         size_t batch) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if ((page_ids == nullptr) != (slots_in_page == nullptr)) return ctx->fail(MLC_ERR_INVALID_ARG, "page_ids and slots_in_page go together");
    PlanKey key = plan->key;   // same shape, new tables
    key.batch = batch;
    int st = validate_tables(ctx, key, nullptr, page_tables_flat, n_page_tables_flat, page_table_offsets, seq_lens,
                             q_positions, plan->key.capacity);
    if (st != MLC_OK) return st;
    if (page_ids)
        for (size_t r = 0; r < batch; ++r) {
            if (key.capacity && page_ids[r] >= key.capacity)
                return ctx->fail(MLC_ERR_BOUNDS, "page_ids[%zu]=%u >= capacity %zu", r, page_ids[r], key.capacity);
            if (slots_in_page[r] >= key.P)
                return ctx->fail(MLC_ERR_BOUNDS, "slots_in_page[%zu]=%u >= page size", r, slots_in_page[r]);
        }
    DeviceGuard guard(ctx->device);
    plan->key = key;
    // the rebuild waits for the previous upload to have left the pinned staging copy; the device copy is
    // overwritten in stream order, after the kernels already enqueued with the old tables
    return build_plan(ctx, *plan, page_tables_flat, page_table_offsets, seq_lens, q_positions, page_ids, slots_in_page);
}

void mlc_attn_plan_destroy(mlc_ctx* ctx, mlc_attn_plan* plan) {
    if (!ctx || !plan) return;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    release_plan_buffers(*plan);
    delete plan;
}

int mlc_encode_paged_flash_attention_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                             const void* k_pages, const void* v_pages, void* o,
                                             float scale, int q_dtype, int o_dtype) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    return launch_with_plan(ctx, a, *plan);
}

}  // extern "C"

namespace mlcb {
// mlc_encode_paged_flash_attention_planned for a caller that knows what the kernel in front wrote (see
// AttnArgs::only_plan_rows_written): the walker's decode pass, whose QKV projection writes the newest token's rows.
int encode_attention_planned_after_row_write(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q, const void* k_pages,
                                             const void* v_pages, void* o, float scale, int q_dtype, int o_dtype) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    a.only_plan_rows_written = true;
    return launch_with_plan(ctx, a, *plan);
}
}  // namespace mlcb

extern "C" {

int mlc_encode_paged_attention_partial_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                               const void* k_pages, const void* v_pages,
                                               float* o_partial, float* ml_partial, float scale,
                                               int q_dtype) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!o_partial || !ml_partial) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages;
    a.o_partial = o_partial; a.ml_partial = ml_partial;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = MLC_F32;
    return launch_with_plan(ctx, a, *plan);
}

int mlc_encode_paged_attention_exchange_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, mlc_exchange* ex, const void* q,
                                                const void* k_pages, const void* v_pages, void* out, float scale,
                                                int q_dtype, int o_dtype) {
    if (!ctx || !plan || !ex) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!q || !k_pages || !v_pages || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if ((q_dtype != MLC_F32 && q_dtype != MLC_F16) || (o_dtype != MLC_F32 && o_dtype != MLC_F16))
        return ctx->fail(MLC_ERR_INVALID_ARG, "dtype must be MLC_F32 or MLC_F16");
    ExchangeView xv;
    if (!exchange_describe(ex, &xv)) return ctx->fail(MLC_ERR_INVALID_ARG, "exchange not attached to its peers");
    const PlanKey& k = plan->key;
    const size_t rows = k.batch * k.H;
    if (rows == 0 || rows > xv.max_rows || xv.D != k.D)
        return ctx->fail(MLC_ERR_INVALID_ARG, "the exchange was created for %zu rows of head_dim %zu, the plan has %zu of %zu",
                         xv.max_rows, xv.D, rows, k.D);
    if (reinterpret_cast<uintptr_t>(out) % 16) return ctx->fail(MLC_ERR_INVALID_ARG, "out must be 16-byte aligned");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    a.batch = k.batch; a.H = k.H; a.KVH = k.KVH; a.D = k.D; a.P = k.P; a.capacity = k.capacity;
    if (a.scale <= 0.f) a.scale = 1.0f / std::sqrt(static_cast<float>(a.D));  // mm:7133
    AttnArgs probe = a;
    probe.o = out;
    if (plan->view.has_tma && plan->view.unit_mode && plan->view.hpc <= 1 && !ctx->force_general && k.D % 4 == 0 &&
        decode_tma_pointers_supported(probe)) {
        a.exchange = &xv;
        a.exchange_out = out;
        ctx->last_attention_kernel = 2;
        return launch_attention_decode_tma(ctx, a, plan->view);
    }
    // Any other plan (split form, odd shapes): the partial into scratch kept by the context, then the
    // separate exchange + combine kernel.
    const size_t o_bytes = rows * k.D * 4, ml_bytes = rows * 2 * 4;
    char* scratch = static_cast<char*>(mlc_cached_buffer(ctx, "mlc_exchange_partials", ((o_bytes + 255) / 256) * 256 + ml_bytes));
    if (!scratch) return ctx->fail(MLC_ERR_OOM, "scratch for the partials unavailable");
    float* o_partial = reinterpret_cast<float*>(scratch);
    float* ml_partial = reinterpret_cast<float*>(scratch + ((o_bytes + 255) / 256) * 256);
    int st = mlc_encode_paged_attention_partial_planned(ctx, plan, q, k_pages, v_pages, o_partial, ml_partial, scale, q_dtype);
    if (st != MLC_OK) return st;
    return mlc_encode_exchange_lse_combine(ctx, ex, o_partial, ml_partial, rows, out, o_dtype);
}

int mlc_encode_paged_decode_step_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                         const void* k_new, const void* v_new, void* k_pages,
                                         void* v_pages, void* o, float scale, int q_dtype, int o_dtype) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!plan->d_page_ids) return ctx->fail(MLC_ERR_INVALID_ARG, "the plan was created without page_ids / slots_in_page");
    if (!k_new || !v_new || !k_pages || !v_pages) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    a.k_new = k_new; a.v_new = v_new;
    const PlanKey& k = plan->key;
    if (plan->view.step_fusable && !ctx->force_general && decode_tma_pointers_supported(a))
        return launch_with_plan(ctx, a, *plan);
    // not fusable (odd shape, causal cut before the newest token, unaligned buffers): two launches
    int st = launch_scatter_rows_device_tables(ctx, k_pages, v_pages, plan->d_page_ids, plan->d_slots, k.P,
                                               k.KVH, k.D, k.batch, k_new, v_new, k.capacity);
    if (st != MLC_OK) return st;
    a.k_new = a.v_new = nullptr;
    return launch_with_plan(ctx, a, *plan);
}

int mlc_encode_paged_decode_pass_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, size_t n_layers,
                                         const void* const* q, const void* const* k_new,
                                         const void* const* v_new, void* const* k_pages, void* const* v_pages,
                                         void* const* o, float scale, int q_dtype, int o_dtype) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!q || !k_new || !v_new || !k_pages || !v_pages || !o) return ctx->fail(MLC_ERR_INVALID_ARG, "null pointer array");
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    // One launch for the whole pass when the plan keeps every (request, head) inside a CTA: the layers of
    // this call are independent of one another by contract (all their inputs are given up front), so their
    // work items can be dealt to the CTAs across layers. MLC_B200_DECODE_PASS=0 keeps one launch per layer.
    static const bool pass_allowed = env_int("MLC_B200_DECODE_PASS", 1) != 0;
    if (pass_allowed && !ctx->force_general && decode_pass_supported(plan->view_pass, n_layers) &&
        (q_dtype == MLC_F32 || q_dtype == MLC_F16) && (o_dtype == MLC_F32 || o_dtype == MLC_F16)) {
        DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
        const PlanKey& k = plan->key;
        AttnArgs shape;
        shape.batch = k.batch; shape.H = k.H; shape.KVH = k.KVH; shape.D = k.D; shape.P = k.P; shape.capacity = k.capacity;
        shape.scale = scale > 0.f ? scale : 1.0f / std::sqrt(static_cast<float>(k.D));  // mm:7133
        shape.q_dtype = q_dtype; shape.o_dtype = o_dtype;
        const int st = launch_decode_pass_tma(ctx, shape, plan->view_pass, n_layers, q, k_new, v_new, k_pages, v_pages, o);
        if (st == MLC_OK) ctx->last_attention_kernel = 2;
        if (st != MLC_ERR_UNSUPPORTED) return st;
    }
    for (size_t l = 0; l < n_layers; ++l) {
        const int st = mlc_encode_paged_decode_step_planned(ctx, plan, q[l], k_new[l], v_new[l], k_pages[l], v_pages[l],
                                                            o[l], scale, q_dtype, o_dtype);
        if (st != MLC_OK) return st;
    }
    return MLC_OK;
}

int mlc_encode_paged_decode_pass_host(mlc_ctx* ctx, const mlc_attn_plan* plan, size_t n_layers, const void* host_in,
                                      void* dev_in, void* const* k_pages, void* const* v_pages, void* dev_o,
                                      void* host_o, float scale, int q_dtype, int o_dtype, size_t n_groups) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (ctx->capturing) return ctx->fail(MLC_ERR_UNSUPPORTED, "the host-buffer pass uses its own copy streams and cannot be captured");
    if (!host_in || !dev_in || !k_pages || !v_pages || !dev_o || !host_o || !n_layers) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if ((q_dtype != MLC_F16 && q_dtype != MLC_F32) || (o_dtype != MLC_F16 && o_dtype != MLC_F32))
        return ctx->fail(MLC_ERR_INVALID_ARG, "q / o dtype must be MLC_F16 or MLC_F32");
    const PlanKey& k = plan->key;
    const size_t q_bytes = k.batch * k.H * k.D * (q_dtype == MLC_F32 ? 4 : 2);
    const size_t kv_bytes = k.batch * k.KVH * k.D * 2;
    const size_t in_row = q_bytes + 2 * kv_bytes;
    const size_t o_row = k.batch * k.H * k.D * (o_dtype == MLC_F32 ? 4 : 2);
    if (in_row % 16 || q_bytes % 16 || kv_bytes % 16) return ctx->fail(MLC_ERR_UNSUPPORTED, "rows of the packed input must be multiples of 16 bytes");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    // Zero-copy form: when the whole pass can be one launch and both host buffers are pinned memory the GPU can
    // address, the kernel reads Q and the new rows straight from host memory (each row once, a work item
    // ahead of its use) and writes O straight into it, so the transfers run inside the kernel, beside the KV
    // stream, instead of in front of and behind it. MLC_B200_DECODE_ZERO_COPY=0 keeps the copy pipeline below.
    static const int zero_copy_mode = env_int("MLC_B200_DECODE_PASS", 1) != 0 ? env_int("MLC_B200_DECODE_ZERO_COPY", 1) : 0;
    if (zero_copy_mode != 0 && !ctx->force_general && decode_pass_supported(plan->view_pass, n_layers)) {
        cudaPointerAttributes ai{}, ao{};
        const bool mapped = cudaPointerGetAttributes(&ai, host_in) == cudaSuccess && ai.type == cudaMemoryTypeHost && ai.devicePointer &&
                            cudaPointerGetAttributes(&ao, host_o) == cudaSuccess && ao.type == cudaMemoryTypeHost && ao.devicePointer;
        cudaGetLastError();   // a pointer the runtime does not know is not an error here
        if (mapped) {
            if (ctx->host_pass_done) {   // an earlier host-buffer pass of the copying form may still read dev_o
                MLCB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->host_pass_done, 0));
                ctx->host_pass_done = nullptr;
            }
            const char* gin = static_cast<const char*>(ai.devicePointer);
            char* gout = static_cast<char*>(ao.devicePointer);
            if (zero_copy_mode == 2) {   // experiment: inputs by one bulk copy, outputs written by the kernel
                MLCB_CUDA(ctx, cudaMemcpyAsync(dev_in, host_in, n_layers * in_row, cudaMemcpyHostToDevice, ctx->stream));
                gin = static_cast<const char*>(dev_in);
            } else if (zero_copy_mode == 3) {   // experiment: inputs read by the kernel, outputs by one bulk copy
                gout = static_cast<char*>(dev_o);
            }
            const void* qv[kMaxPassLayersApi];
            const void* knv[kMaxPassLayersApi];
            const void* vnv[kMaxPassLayersApi];
            void* ov[kMaxPassLayersApi];
            for (size_t l = 0; l < n_layers; ++l) {
                qv[l] = gin + l * in_row;
                knv[l] = gin + l * in_row + q_bytes;
                vnv[l] = gin + l * in_row + q_bytes + kv_bytes;
                ov[l] = gout + l * o_row;
            }
            AttnArgs shape;
            shape.batch = k.batch; shape.H = k.H; shape.KVH = k.KVH; shape.D = k.D; shape.P = k.P; shape.capacity = k.capacity;
            shape.scale = scale > 0.f ? scale : 1.0f / std::sqrt(static_cast<float>(k.D));  // mm:7133
            shape.q_dtype = q_dtype; shape.o_dtype = o_dtype;
            const int st = launch_decode_pass_tma(ctx, shape, plan->view_pass, n_layers, qv, knv, vnv, k_pages, v_pages, ov);
            if (st == MLC_OK) ctx->last_attention_kernel = 2;
            if (st == MLC_OK && zero_copy_mode == 3)
                MLCB_CUDA(ctx, cudaMemcpyAsync(host_o, dev_o, n_layers * o_row, cudaMemcpyDeviceToHost, ctx->stream));
            if (st != MLC_ERR_UNSUPPORTED) return st;
        }
    }
    // group boundaries: two layers first and last (little copy time left uncovered), the rest in equal parts
    std::vector<size_t> bounds;
    if (n_groups == 0) n_groups = 5;
    if (n_groups >= 3 && n_layers >= 2 * n_groups) {
        bounds.push_back(0);
        const size_t mid = n_layers - 4, parts = n_groups - 2;
        for (size_t i = 0; i <= parts; ++i) bounds.push_back(2 + mid * i / parts);
        bounds.push_back(n_layers);
    } else {
        n_groups = std::min(n_groups, n_layers);
        for (size_t i = 0; i <= n_groups; ++i) bounds.push_back(n_layers * i / n_groups);
    }
    const size_t G = bounds.size() - 1;
    if (!ctx->h2d_stream) {
        MLCB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
        MLCB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
    }
    while (ctx->pass_events.size() < 2 * G + 2) {
        cudaEvent_t e;
        MLCB_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->pass_events.push_back(e);
    }
    cudaEvent_t ev_start = ctx->pass_events[2 * G], ev_done = ctx->pass_events[2 * G + 1];
    // a previous host-buffer pass that was not flushed: its copies back still read dev_o
    if (ctx->host_pass_done) {
        MLCB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->host_pass_done, 0));
        ctx->host_pass_done = nullptr;
    }
    // the staging buffer may still be read by kernels already in the stream
    MLCB_CUDA(ctx, cudaEventRecord(ev_start, ctx->stream));
    MLCB_CUDA(ctx, cudaStreamWaitEvent(ctx->h2d_stream, ev_start, 0));
    const char* hin = static_cast<const char*>(host_in);
    char* din = static_cast<char*>(dev_in);
    char* dout = static_cast<char*>(dev_o);
    char* hout = static_cast<char*>(host_o);
    for (size_t g = 0; g < G; ++g) {
        const size_t a = bounds[g], b = bounds[g + 1];
        MLCB_CUDA(ctx, cudaMemcpyAsync(din + a * in_row, hin + a * in_row, (b - a) * in_row, cudaMemcpyHostToDevice, ctx->h2d_stream));
        MLCB_CUDA(ctx, cudaEventRecord(ctx->pass_events[g], ctx->h2d_stream));
    }
    for (size_t g = 0; g < G; ++g) {
        const size_t a = bounds[g], b = bounds[g + 1];
        MLCB_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->pass_events[g], 0));
        for (size_t l = a; l < b; ++l) {
            const char* row = din + l * in_row;
            const int st = mlc_encode_paged_decode_step_planned(ctx, plan, row, row + q_bytes, row + q_bytes + kv_bytes, k_pages[l],
                                                                v_pages[l], dout + l * o_row, scale, q_dtype, o_dtype);
            if (st != MLC_OK) return st;
        }
        MLCB_CUDA(ctx, cudaEventRecord(ctx->pass_events[G + g], ctx->stream));
        MLCB_CUDA(ctx, cudaStreamWaitEvent(ctx->d2h_stream, ctx->pass_events[G + g], 0));
        MLCB_CUDA(ctx, cudaMemcpyAsync(hout + a * o_row, dout + a * o_row, (b - a) * o_row, cudaMemcpyDeviceToHost, ctx->d2h_stream));
    }
    // mlc_pass_flush waits for this event after the context's stream; the stream itself is not held
    // up by the last copy back, so what the caller queues next (a plan update's upload) runs beside it
    MLCB_CUDA(ctx, cudaEventRecord(ev_done, ctx->d2h_stream));
    ctx->host_pass_done = ev_done;
    return MLC_OK;
}

int mlc_encode_scatter_kv_pair_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, void* k_page_storage,
                                       void* v_page_storage, const void* k_src, const void* v_src) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!plan->d_page_ids) return ctx->fail(MLC_ERR_INVALID_ARG, "the plan was created without page_ids / slots_in_page");
    if (!k_page_storage || !v_page_storage || !k_src || !v_src) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    const PlanKey& k = plan->key;
    return launch_scatter_rows_device_tables(ctx, k_page_storage, v_page_storage, plan->d_page_ids,
                                             plan->d_slots, k.P, k.KVH, k.D, k.batch, k_src, v_src, k.capacity);
}

int mlc_encode_qkv_split_rope_scatter_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* qkv,
                                              void* q_out, int q_dtype, void* k_page_storage,
                                              void* v_page_storage, const void* cos_table,
                                              const void* sin_table, size_t qkv_rows, size_t rotary_dim) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!plan->d_page_ids) return ctx->fail(MLC_ERR_INVALID_ARG, "the plan was created without page_ids / slots_in_page");
    if (!q_out || !k_page_storage || !v_page_storage) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (q_dtype != MLC_F16 && q_dtype != MLC_F32) return ctx->fail(MLC_ERR_INVALID_ARG, "q dtype must be MLC_F16 or MLC_F32");
    const PlanKey& k = plan->key;
    int st = check_qkv_rope_args(ctx, qkv, cos_table, sin_table, k.batch, k.H, k.KVH, k.D, qkv_rows, k.H * k.D,
                                 k.KVH * k.D, k.KVH * k.D, rotary_dim);
    if (st != MLC_OK) return st;
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    QkvRopeParams p{};
    p.qkv = static_cast<const float*>(qkv);
    if (q_dtype == MLC_F32) p.q = static_cast<float*>(q_out);
    else p.q16 = static_cast<__half*>(q_out);
    p.k_pool = static_cast<__half*>(k_page_storage);
    p.v_pool = static_cast<__half*>(v_page_storage);
    p.page_ids = plan->d_page_ids;
    p.slots = plan->d_slots;
    p.cos_t = static_cast<const float*>(cos_table);
    p.sin_t = static_cast<const float*>(sin_table);
    p.err = ctx->d_err;
    p.batch = static_cast<uint32_t>(k.batch);
    p.head_dim = static_cast<uint32_t>(k.D);
    p.rotary_pairs = static_cast<uint32_t>(rotary_dim / 2);
    p.qkv_rows = static_cast<uint32_t>(qkv_rows);
    p.q_rows = static_cast<uint32_t>(k.H * k.D);
    p.k_rows = p.v_rows = static_cast<uint32_t>(k.KVH * k.D);
    p.page_tokens = static_cast<uint32_t>(k.P);
    p.capacity = k.capacity ? static_cast<uint32_t>(k.capacity) : 0xFFFFFFFFu;
    return launch_qkv_split_rope_cast(ctx, p);
}

int mlc_encode_matmul_qkv_rope_scatter_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, int quant, const void* weights,
                                               const void* in, size_t in_stride, int input_kind, size_t cols,
                                               size_t row_stride, void* q_out, void* k_page_storage,
                                               void* v_page_storage, const void* cos_table, const void* sin_table,
                                               size_t rotary_dim) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!plan->d_page_ids) return ctx->fail(MLC_ERR_INVALID_ARG, "the plan was created without page_ids / slots_in_page");
    if (!q_out || !k_page_storage || !v_page_storage) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    const PlanKey& k = plan->key;
    const size_t qkv_rows = (k.H + 2 * k.KVH) * k.D;
    // `in` stands in for the qkv buffer of the unfused form in the shared argument check (pointer and alignment only)
    int st = check_qkv_rope_args(ctx, in, cos_table, sin_table, k.batch, k.H, k.KVH, k.D, qkv_rows, k.H * k.D, k.KVH * k.D,
                                 k.KVH * k.D, rotary_dim);
    if (st != MLC_OK) return st;
    DeviceGuard guard(ctx->device);
    if (int ust = use_plan(ctx, plan); ust != MLC_OK) return ust;
    QkvRopeParams p{};
    p.q16 = static_cast<__half*>(q_out);
    p.k_pool = static_cast<__half*>(k_page_storage);
    p.v_pool = static_cast<__half*>(v_page_storage);
    p.page_ids = plan->d_page_ids;
    p.slots = plan->d_slots;
    p.cos_t = static_cast<const float*>(cos_table);
    p.sin_t = static_cast<const float*>(sin_table);
    p.err = ctx->d_err;
    p.batch = static_cast<uint32_t>(k.batch);
    p.head_dim = static_cast<uint32_t>(k.D);
    p.rotary_pairs = static_cast<uint32_t>(rotary_dim / 2);
    p.qkv_rows = static_cast<uint32_t>(qkv_rows);
    p.q_rows = static_cast<uint32_t>(k.H * k.D);
    p.k_rows = p.v_rows = static_cast<uint32_t>(k.KVH * k.D);
    p.page_tokens = static_cast<uint32_t>(k.P);
    p.capacity = k.capacity ? static_cast<uint32_t>(k.capacity) : 0xFFFFFFFFu;
    return encode_matvec_qkv_rope(ctx, quant, input_kind, weights, in, in_stride, cols, row_stride, p);
}

}  // extern "C"
