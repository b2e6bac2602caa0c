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

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace mlcb {

namespace {

struct PlanKey {
    size_t batch = 0, H = 0, KVH = 0, D = 0, P = 0, capacity = 0, n_flat = 0;
    int causal = 0;
    bool tma = false;
    bool operator==(const PlanKey& o) const {
        return batch == o.batch && H == o.H && KVH == o.KVH && D == o.D && P == o.P &&
               capacity == o.capacity && n_flat == o.n_flat && causal == o.causal && tma == o.tma;
    }
};

struct PlanEntry {
    PlanKey key;
    std::vector<uint32_t> tables;  // pt_flat | pt_off | seq_lens | q_pos as passed by the caller
    uint8_t* host = nullptr;       // pinned image of the device blob
    uint8_t* dev = nullptr;
    size_t cap = 0;
    cudaEvent_t uploaded = nullptr;
    DecodePlanView view;
    uint64_t stamp = 0;
};

}  // namespace

struct AttnPlanCache {
    static constexpr int kEntries = 4;
    PlanEntry e[kEntries];
    uint64_t clock = 0;
};

void destroy_plan_cache(mlc_ctx* ctx) {
    if (!ctx->plan_cache) return;
    for (auto& p : ctx->plan_cache->e) {
        if (p.host) cudaFreeHost(p.host);
        if (p.dev) cudaFree(p.dev);
        if (p.uploaded) cudaEventDestroy(p.uploaded);
    }
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
int build_plan(mlc_ctx* ctx, PlanEntry& p, const uint32_t* pt_flat, const uint32_t* pt_off,
               const uint32_t* seq_lens, const uint32_t* q_pos) {
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

    std::vector<uint32_t> counts;
    std::vector<std::vector<PieceDesc>> cta_pieces;
    std::vector<std::vector<uint32_t>> cta_tiles;
    uint32_t n_cta = 0, max_pieces = 1, max_tiles = 1, n_slots = 0, n_segs = 0;
    if (k.tma) {
        const uint32_t TOK = kTileTokens;
        const uint32_t n_hb = static_cast<uint32_t>((k.KVH + kDecodeWarps - 1) / kDecodeWarps);
        uint64_t total = 0;
        for (size_t r = 0; r < N; ++r) total += static_cast<uint64_t>((eff[r] + TOK - 1) / TOK) * n_hb;
        int per_sm = env_int("MLC_B200_DECODE_CTAS_PER_SM", k.D <= 64 ? 2 : 1);
        uint64_t max_cta = static_cast<uint64_t>(ctx->sm_count) * std::max(per_sm, 1);
        int min_tiles = std::max(env_int("MLC_B200_DECODE_MIN_TILES", 1), 1);
        n_cta = static_cast<uint32_t>(std::max<uint64_t>(1, std::min<uint64_t>(max_cta, total / min_tiles)));
        cta_pieces.resize(n_cta);
        cta_tiles.resize(n_cta);
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
                    seg_pieces.emplace_back(c, static_cast<uint32_t>(cta_pieces[c].size()));
                    cta_pieces[c].push_back(d);
                    for (uint32_t i = 0; i < take; ++i) {
                        // tile word: page id | sub-tile within the page << 25 | head block << 28
                        uint64_t tok0 = static_cast<uint64_t>(t + i) * TOK;
                        uint32_t page = pt_flat[pt_off[r] + tok0 / k.P];
                        uint32_t sub = static_cast<uint32_t>((tok0 % k.P) / TOK);
                        cta_tiles[c].push_back(page | (sub << 25) | (hb << 28));
                    }
                    t += take;
                    g += take;
                }
                uint16_t parts = static_cast<uint16_t>(seg_pieces.size());
                uint32_t first_slot = n_slots;
                for (size_t i = 0; i < seg_pieces.size(); ++i) {
                    PieceDesc& d = cta_pieces[seg_pieces[i].first][seg_pieces[i].second];
                    d.n_parts = parts;
                    d.seg = parts > 1 ? n_segs : 0;
                    d.seg_first_slot = first_slot;
                    d.part_slot = first_slot + static_cast<uint32_t>(i);
                }
                if (parts > 1) {
                    n_slots += parts;
                    ++n_segs;
                }
            }
        }
        for (uint32_t i = 0; i < n_cta; ++i) {
            max_pieces = std::max<uint32_t>(max_pieces, static_cast<uint32_t>(cta_pieces[i].size()));
            max_tiles = std::max<uint32_t>(max_tiles, static_cast<uint32_t>(cta_tiles[i].size()));
        }
    }

    // ---- lay the image out
    size_t off = 0;
    const size_t off_counts = off;   off = align_up(off + size_t(n_cta) * 8, 16);
    const size_t off_pieces = off;   off = align_up(off + size_t(n_cta) * max_pieces * sizeof(PieceDesc), 16);
    const size_t off_tiles = off;    off = align_up(off + size_t(n_cta) * max_tiles * 4, 16);
    const size_t off_flat = off;     off = align_up(off + k.n_flat * 4, 16);
    const size_t off_ptoff = off;    off = align_up(off + (N + 1) * 4, 16);
    const size_t off_eff = off;      off = align_up(off + N * 4, 16);
    const size_t off_zero = off;     off = align_up(off + zero_rows.size() * 4, 16);
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
    }
    if (!p.uploaded) MLCB_CUDA(ctx, cudaEventCreateWithFlags(&p.uploaded, cudaEventDisableTiming));

    std::memset(p.host, 0, bytes);
    auto* counts_h = reinterpret_cast<uint32_t*>(p.host + off_counts);
    auto* pieces_h = reinterpret_cast<PieceDesc*>(p.host + off_pieces);
    auto* tiles_h = reinterpret_cast<uint32_t*>(p.host + off_tiles);
    for (uint32_t i = 0; i < n_cta; ++i) {
        counts_h[2 * i] = static_cast<uint32_t>(cta_pieces[i].size());
        counts_h[2 * i + 1] = static_cast<uint32_t>(cta_tiles[i].size());
        std::copy(cta_pieces[i].begin(), cta_pieces[i].end(), pieces_h + size_t(i) * max_pieces);
        std::copy(cta_tiles[i].begin(), cta_tiles[i].end(), tiles_h + size_t(i) * max_tiles);
    }
    std::memcpy(p.host + off_flat, pt_flat, k.n_flat * 4);
    std::memcpy(p.host + off_ptoff, pt_off, (N + 1) * 4);
    std::memcpy(p.host + off_eff, eff.data(), N * 4);
    if (!zero_rows.empty()) std::memcpy(p.host + off_zero, zero_rows.data(), zero_rows.size() * 4);
    MLCB_CUDA(ctx, cudaMemcpyAsync(p.dev, p.host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    MLCB_CUDA(ctx, cudaEventRecord(p.uploaded, ctx->stream));

    DecodePlanView& v = p.view;
    v.cta_counts = reinterpret_cast<const uint32_t*>(p.dev + off_counts);
    v.pieces = reinterpret_cast<const PieceDesc*>(p.dev + off_pieces);
    v.tile_pages = reinterpret_cast<const uint32_t*>(p.dev + off_tiles);
    v.pt_flat = reinterpret_cast<const uint32_t*>(p.dev + off_flat);
    v.pt_off = reinterpret_cast<const uint32_t*>(p.dev + off_ptoff);
    v.eff_len = reinterpret_cast<const uint32_t*>(p.dev + off_eff);
    v.zero_rows = reinterpret_cast<const uint32_t*>(p.dev + off_zero);
    v.n_cta = n_cta;
    v.max_pieces = max_pieces;
    v.max_tiles = max_tiles;
    v.n_zero = static_cast<uint32_t>(zero_rows.size());
    v.n_slots = n_slots;
    v.n_segs = n_segs;
    return MLC_OK;
}

int get_plan(mlc_ctx* ctx, const PlanKey& key, const uint32_t* pt_flat, const uint32_t* pt_off,
             const uint32_t* seq_lens, const uint32_t* q_pos, const DecodePlanView** out) {
    if (!ctx->plan_cache) ctx->plan_cache = new AttnPlanCache();
    AttnPlanCache& pc = *ctx->plan_cache;
    const size_t N = key.batch;
    const size_t words = key.n_flat + (N + 1) + N + N;
    PlanEntry* victim = &pc.e[0];
    for (auto& p : pc.e) {
        if (p.stamp && p.key == key && p.tables.size() == words) {
            const uint32_t* t = p.tables.data();
            if (!std::memcmp(t, pt_flat, key.n_flat * 4) &&
                !std::memcmp(t + key.n_flat, pt_off, (N + 1) * 4) &&
                !std::memcmp(t + key.n_flat + N + 1, seq_lens, N * 4) &&
                !std::memcmp(t + key.n_flat + 2 * N + 1, q_pos, N * 4)) {
                p.stamp = ++pc.clock;
                *out = &p.view;
                return MLC_OK;
            }
        }
        if (p.stamp < victim->stamp) victim = &p;
    }
    PlanEntry& p = *victim;
    p.key = key;
    p.tables.resize(words);
    std::memcpy(p.tables.data(), pt_flat, key.n_flat * 4);
    std::memcpy(p.tables.data() + key.n_flat, pt_off, (N + 1) * 4);
    std::memcpy(p.tables.data() + key.n_flat + N + 1, seq_lens, N * 4);
    std::memcpy(p.tables.data() + key.n_flat + 2 * N + 1, q_pos, N * 4);
    p.stamp = 0;
    int st = build_plan(ctx, p, pt_flat, pt_off, seq_lens, q_pos);
    if (st != MLC_OK) return st;
    p.stamp = ++pc.clock;
    *out = &p.view;
    return MLC_OK;
}

int attention_impl(mlc_ctx* ctx, bool sync, AttnArgs a, const uint32_t* pt_flat, size_t n_flat,
                   const uint32_t* pt_off, const uint32_t* seq_lens, const uint32_t* q_pos,
                   int causal, size_t capacity_pages) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    // metal_runtime.mm:7742-7750
    if (!a.q || !a.k_pages || !a.v_pages || (!a.o && !a.o_partial))
        return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (a.batch == 0 || a.H == 0 || a.D == 0 || a.P == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (a.KVH == 0 || a.H % a.KVH != 0) return ctx->fail(MLC_ERR_INVALID_ARG, "num_heads must be a multiple of kv_heads");
    if (!pt_off || !seq_lens || !q_pos || (!pt_flat && n_flat)) return ctx->fail(MLC_ERR_INVALID_ARG, "null table");
    if (n_flat < pt_off[a.batch]) return ctx->fail(MLC_ERR_INVALID_ARG, "page_tables_flat shorter than the last offset");
    if (a.D > 256) return ctx->fail(MLC_ERR_UNSUPPORTED, "head_dim > 256");
    if ((a.q_dtype != MLC_F32 && a.q_dtype != MLC_F16) || (a.o_dtype != MLC_F32 && a.o_dtype != MLC_F16))
        return ctx->fail(MLC_ERR_INVALID_ARG, "dtype must be MLC_F32 or MLC_F16");
    if (!sync && !ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (a.batch * a.H >= (size_t(1) << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch * heads too large");
    // checks the reference does not make
    a.capacity = resolve_capacity(ctx, a.k_pages, capacity_pages, a.P * a.KVH * a.D * 2);
    for (size_t r = 0; r < a.batch; ++r) {
        if (pt_off[r + 1] < pt_off[r]) return ctx->fail(MLC_ERR_BOUNDS, "page_table_offsets not monotone at %zu", r);
        uint64_t room = static_cast<uint64_t>(pt_off[r + 1] - pt_off[r]) * a.P;
        if (seq_lens[r] > room)
            return ctx->fail(MLC_ERR_BOUNDS, "seq_lens[%zu]=%u exceeds its %u pages", r, seq_lens[r], pt_off[r + 1] - pt_off[r]);
    }
    if (a.capacity)
        for (size_t i = 0; i < pt_off[a.batch]; ++i)
            if (pt_flat[i] >= a.capacity)
                return ctx->fail(MLC_ERR_BOUNDS, "page_tables_flat[%zu]=%u >= capacity %zu", i, pt_flat[i], a.capacity);
    if (a.scale <= 0.f) a.scale = 1.0f / std::sqrt(static_cast<float>(a.D));  // mm:7133

    DeviceGuard guard(ctx->device);
    PlanKey key;
    key.batch = a.batch; key.H = a.H; key.KVH = a.KVH; key.D = a.D; key.P = a.P;
    key.capacity = a.capacity; key.n_flat = pt_off[a.batch]; key.causal = causal ? 1 : 0;
    key.tma = !ctx->force_general && decode_tma_supported(ctx, a);
    const DecodePlanView* plan = nullptr;
    int st = get_plan(ctx, key, pt_flat, pt_off, seq_lens, q_pos, &plan);
    if (st != MLC_OK) return st;
    if (key.tma) st = launch_attention_decode_tma(ctx, a, *plan);
    else if (a.o_partial) return ctx->fail(MLC_ERR_UNSUPPORTED, "partial output needs the split-KV kernel's shapes");
    else st = launch_attention_general(ctx, a, plan->pt_flat, plan->pt_off, plan->eff_len);
    if (st != MLC_OK) return st;
    if (sync) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return ctx->fail(MLC_ERR_CUDA, "attention failed: %s", cudaGetErrorString(e));
        uint32_t word = 0;
        MLCB_CUDA(ctx, cudaMemcpy(&word, ctx->d_err, 4, cudaMemcpyDeviceToHost));
        if (word) {
            cudaMemset(ctx->d_err, 0, 4);
            return ctx->fail(MLC_ERR_DEVICE_FLAG, "attention kernel recorded error word 0x%x", word);
        }
    }
    return MLC_OK;
}

}  // namespace
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

}  // extern "C"
