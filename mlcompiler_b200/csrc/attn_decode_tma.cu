// Split-KV paged decode attention for sm_100a: TMA-staged pages, tensor-core dots.
//
// Computes what the reference's MSL kernel paged_flash_attention computes
// (compiler/runtime/metal_runtime.mm:2216-2335) with a different decomposition:
//
//   reference                               here
//   ---------------------------------------------------------------------------
//   one threadgroup per (request, q head):  one warp per (request, KV head, run of
//   every q head of a GQA group re-reads    tiles): the G = H/KVH query heads of a
//   the same K/V rows (G x the traffic)     group share each K/V byte read from HBM
//   whole sequence walked by one group      persistent grid; the (request, head
//                                           block, tile) sequence is cut into equal
//                                           contiguous runs, one per CTA, so a long
//                                           request is split over many CTAs and
//                                           short ones share a CTA (flash-decoding)
//   element-wise page-indirected loads      one TMA box per (page, KV head, 32
//   widened to fp32 in threadgroup memory   tokens): 32 rows x 128 B, 128B-swizzled,
//                                           into a per-warp ring of shared-memory
//                                           stages guarded by mbarriers
//   D-long scalar dot per thread, tree      mma.sync m16n8k16 (fp16 in, fp32
//   reductions through threadgroup memory   accumulate) for Q.K^T and P.V; row max
//                                           and row sum by quad shuffles
//
// G = 8 means 4 FMA per KV byte; at HBM speed that is more than half of the
// SM's fp32 FMA rate before any fp16->fp32 conversion, so the dots go through the
// tensor cores and the kernel stays bandwidth-bound. tcgen05/TMEM is not used
// here: a decode tile has 8 (or 4) query rows against the 64-row minimum of a
// tcgen05 MMA, and the accumulators fit in registers.
//
// Partials of a (request, KV head) that is split over several CTAs go to a
// workspace as un-normalised (o, m, l); the warp that arrives last (an atomic
// counter, no waiting) merges them with the log-sum-exp rule and writes O.
//
// Nothing here spins on another CTA. The only waits are mbarrier waits on this
// warp's own TMA copies; they are bounded, and on expiry the warp records
// MLC_DEVERR_WAIT_TIMEOUT and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "attn_internal.hpp"

namespace mlcb {

// ------------------------------------------------------------------------------
// tensor maps
// ------------------------------------------------------------------------------
struct TensorMapCache {
    struct Entry {
        const void* pool;
        size_t D, KVH, P, capacity;
        CUtensorMap map;
    };
    std::vector<Entry> entries;
    void* encode_fn = nullptr;
};

void destroy_tmap_cache(mlc_ctx* ctx) {
    delete ctx->tmap_cache;
    ctx->tmap_cache = nullptr;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Map over one pool viewed as [capacity][P][KVH][D] halfs; box = 64 halfs of one
// KV head for kTileTokens consecutive slots of one page, 128-byte swizzled.
static int get_tensor_map(mlc_ctx* ctx, const void* pool, const AttnArgs& a, const CUtensorMap** out) {
    if (!ctx->tmap_cache) ctx->tmap_cache = new TensorMapCache();
    TensorMapCache& tc = *ctx->tmap_cache;
    for (auto& e : tc.entries)
        if (e.pool == pool && e.D == a.D && e.KVH == a.KVH && e.P == a.P && e.capacity == a.capacity) {
            *out = &e.map;
            return MLC_OK;
        }
    if (!tc.encode_fn) {
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &tc.encode_fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !tc.encode_fn)
            return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    TensorMapCache::Entry e{pool, a.D, a.KVH, a.P, a.capacity, {}};
    cuuint64_t dims[4] = {a.D, a.KVH, a.P, a.capacity};
    cuuint64_t strides[3] = {a.D * 2, a.KVH * a.D * 2, a.P * a.KVH * a.D * 2};
    cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(kTileTokens), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(tc.encode_fn)(
        &e.map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(pool), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    if (tc.entries.size() >= 256) tc.entries.erase(tc.entries.begin());
    tc.entries.push_back(e);
    *out = &tc.entries.back().map;
    return MLC_OK;
}

// ------------------------------------------------------------------------------
// device helpers
// ------------------------------------------------------------------------------
struct DecodeParams {
    const void* q;
    void* o;
    float* o_partial;   // API-level partial output (un-normalised), or null
    float* ml_partial;
    const uint32_t* cta_counts;
    const PieceDesc* pieces;
    const uint32_t* tile_pages;
    const uint32_t* zero_rows;
    float* work_o;      // split-KV workspace: o fragments
    float* work_ml;     // split-KV workspace: (m, l) per lane
    uint32_t* counters;
    uint32_t* err;
    uint32_t max_pieces, max_tiles, n_zero;
    uint32_t H, KVH, G;
    uint32_t stages;
    uint32_t sub_per_page;  // P / kTileTokens
    float scale_log2;       // scale * log2(e)
    int q_f32, o_f32;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: ~2^22 polls (each poll itself suspends for a while) before giving up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 ld_cg_f2(const float2* p) {
    float2 v;
    asm volatile("ld.global.cg.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// Tile entry: page id in bits 0..24, sub-tile within the page in 25..27, head block in 28..31.
static constexpr uint32_t kTilePageMask = (1u << 25) - 1;

// ------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------
template <int D, bool G16>
__global__ void __launch_bounds__(kDecodeWarps * 32)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const DecodeParams prm) {
    constexpr int TOK = kTileTokens;
    constexpr int NT_S = TOK / 8;          // score n-tiles per tile
    constexpr int KSTEPS = D / 16;         // k-steps of Q.K^T
    constexpr int NT_O = D / 8;            // output n-tiles
    constexpr int SUBS = D / 64;           // 64-half boxes per row
    constexpr uint32_t kTileBytes = TOK * D * 2;       // one of K or V
    constexpr uint32_t kStageBytes = 2 * kTileBytes;
    constexpr int ROWSETS = G16 ? 2 : 1;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[kDecodeWarps][8];

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = blockIdx.x;
    const uint32_t stages = prm.stages;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring = smem_base + warp * stages * kStageBytes;

    // Requests that attend to nothing: their O rows are zeros (mm:2254-2257).
    for (uint32_t i = cta; i < prm.n_zero; i += gridDim.x) {
        const uint32_t r = prm.zero_rows[i];
        for (uint32_t e = threadIdx.x; e < prm.H * D; e += blockDim.x) {
            const size_t idx = static_cast<size_t>(r) * prm.H * D + e;
            if (prm.o_partial) {
                prm.o_partial[idx] = 0.f;
                if (e % D == 0) {
                    prm.ml_partial[(idx / D) * 2] = -INFINITY;
                    prm.ml_partial[(idx / D) * 2 + 1] = 0.f;
                }
            } else if (prm.o_f32) static_cast<float*>(prm.o)[idx] = 0.f;
            else static_cast<__half*>(prm.o)[idx] = __float2half_rn(0.f);
        }
    }

    const uint32_t n_pieces = prm.cta_counts[2 * cta];
    const uint32_t n_tiles = prm.cta_counts[2 * cta + 1];
    if (n_tiles == 0) return;
    const uint32_t* my_tiles = prm.tile_pages + static_cast<size_t>(cta) * prm.max_tiles;
    const PieceDesc* my_pieces = prm.pieces + static_cast<size_t>(cta) * prm.max_pieces;

    if (lane == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(smem_u32(&bars[warp][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // Window of 32 tile entries held one per lane.
    uint32_t win_base = 0;
    uint32_t win = (lane < n_tiles) ? __ldg(my_tiles + lane) : 0u;

    auto tile_entry = [&](uint32_t j) -> uint32_t {
        if (j - win_base >= 32u) {  // uniform across the warp
            win_base = j & ~31u;
            win = (win_base + lane < n_tiles) ? __ldg(my_tiles + win_base + lane) : 0u;
        }
        return __shfl_sync(0xffffffffu, win, j - win_base);
    };
    // Ring position counters of this warp. They count only tiles of head blocks in
    // which this warp owns a KV head, in the (identical) order of issue and use.
    uint32_t iss = 0, con = 0;
    // Issues the TMA copies of CTA-local tile j into the next ring stage.
    auto issue = [&](uint32_t j) {
        const uint32_t e = tile_entry(j);
        const uint32_t head = (e >> 28) * kDecodeWarps + warp;
        if (head >= prm.KVH) return;  // this warp has no KV head in that head block
        const uint32_t s = iss % stages;
        ++iss;
        if (lane == 0) {
            const uint32_t bar = smem_u32(&bars[warp][s]);
            const uint32_t dst = ring + s * kStageBytes;
            const int page = static_cast<int>(e & kTilePageMask);
            const int slot0 = static_cast<int>(((e >> 25) & 7u) * TOK);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, kStageBytes);
#pragma unroll
            for (int sub = 0; sub < SUBS; ++sub) {
                tma_load_4d(dst + sub * (TOK * 128), &tmK, bar, sub * 64, static_cast<int>(head), slot0, page);
                tma_load_4d(dst + kTileBytes + sub * (TOK * 128), &tmV, bar, sub * 64, static_cast<int>(head), slot0, page);
            }
        }
    };

    // Prefetches run ahead over piece boundaries; they need nothing but the tile list.
    const uint32_t prologue = n_tiles < stages ? n_tiles : stages;
    for (uint32_t j = 0; j < prologue; ++j) issue(j);

    const uint32_t qrow = lane >> 2, qcol = (lane & 3) * 2;
    uint32_t j = 0;  // CTA-local tile counter (consume side)
    bool dead = false;

    for (uint32_t pi = 0; pi < n_pieces && !dead; ++pi) {
        const uint4 d0 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi));
        const uint4 d1 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi) + 1);
        const uint32_t req = d0.x, piece_tiles = d0.z, part_slot = d0.w;
        const uint32_t seg_first_slot = d1.x, seg = d1.y;
        const uint32_t n_parts = d1.z & 0xffffu, hb = d1.z >> 16;
        const uint32_t last_valid = d1.w & 0xffffu;
        const uint32_t head = hb * kDecodeWarps + warp;
        if (head >= prm.KVH) {  // keep the tile counter and the prefetch stream in step
            for (uint32_t t = 0; t < piece_tiles; ++t, ++j)
                if (j + stages < n_tiles) issue(j + stages);
            continue;
        }

        // ---- Q fragments (A operand), rows = query heads of this KV head's group
        uint32_t qa[KSTEPS][4];
        {
            const size_t q_row0 = (static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G) * D;
#pragma unroll
            for (int rs = 0; rs < 2; ++rs) {
                const uint32_t row = qrow + 8 * rs;
                const bool live = (rs < ROWSETS) && row < prm.G;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t v = 0;
                        if (live) {
                            const size_t idx = q_row0 + static_cast<size_t>(row) * D + kk * 16 + hh * 8 + qcol;
                            if (prm.q_f32) {
                                const float2 f = *reinterpret_cast<const float2*>(static_cast<const float*>(prm.q) + idx);
                                v = pack_half2(f.x, f.y);
                            } else {
                                v = *reinterpret_cast<const uint32_t*>(static_cast<const __half*>(prm.q) + idx);
                            }
                        }
                        qa[kk][rs + 2 * hh] = v;
                    }
                }
            }
        }

        float o_acc[NT_O][4];
#pragma unroll
        for (int n = 0; n < NT_O; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        for (uint32_t t = 0; t < piece_tiles; ++t, ++j) {
            const uint32_t s = con % stages;
            const uint32_t bar = smem_u32(&bars[warp][s]);
            const uint32_t parity = (con / stages) & 1u;
            ++con;
            if (!mbar_wait_bounded(bar, parity)) {
                if (lane == 0) atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT);
                dead = true;
                break;
            }
            const uint32_t sK = ring + s * kStageBytes, sV = sK + kTileBytes;
            const uint32_t nv = (t + 1 == piece_tiles) ? last_valid : TOK;

            // ---- S = Q.K^T (fp32)
            float sc[NT_S][4];
#pragma unroll
            for (int n = 0; n < NT_S; ++n) {
                sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
                const uint32_t tok = n * 8 + (lane & 7);
#pragma unroll
                for (int kp = 0; kp < KSTEPS / 2; ++kp) {
                    const uint32_t chunk = kp * 4 + (lane >> 3);  // 16-byte chunk of the row
                    const uint32_t addr = sK + (chunk >> 3) * (TOK * 128) + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4);
                    uint32_t b[4];
                    ldsm_x4(addr, b);
                    mma_16816(sc[n], qa[2 * kp], b[0], b[1]);
                    mma_16816(sc[n], qa[2 * kp + 1], b[2], b[3]);
                }
            }
            // V rows past the request's last token may hold anything; make them 0 so
            // that 0-weight times garbage cannot produce NaN.
            if (nv < TOK) {
                for (uint32_t i = lane; i < (TOK - nv) * 8 * SUBS; i += 32) {
                    const uint32_t rowi = nv + (i >> 3) % (TOK - nv), sub = (i >> 3) / (TOK - nv);
                    const uint32_t addr = sV + sub * (TOK * 128) + rowi * 128 + ((i & 7) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
                }
                __syncwarp();
            }

            // ---- online softmax on this tile (base-2 domain)
            uint32_t pa[TOK / 16][4];
#pragma unroll
            for (int rs = 0; rs < ROWSETS; ++rs) {
                float tmax = -INFINITY;
#pragma unroll
                for (int n = 0; n < NT_S; ++n) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const uint32_t tok = n * 8 + qcol + e;
                        float v = sc[n][2 * rs + e] * prm.scale_log2;
                        v = tok < nv ? v : -INFINITY;
                        sc[n][2 * rs + e] = v;
                        tmax = fmaxf(tmax, v);
                    }
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run[rs], tmax);  // finite: every tile has >= 1 valid token
                const float alpha = ex2(m_run[rs] - m_new);  // ex2(-inf) = 0 on the first tile
                float psum = 0.f;
#pragma unroll
                for (int n = 0; n < NT_S; ++n) {
                    const float p0 = ex2(sc[n][2 * rs] - m_new), p1 = ex2(sc[n][2 * rs + 1] - m_new);
                    psum += p0 + p1;
                    pa[n >> 1][rs + 2 * (n & 1)] = pack_half2(p0, p1);
                }
                l_run[rs] = l_run[rs] * alpha + psum;
                m_run[rs] = m_new;
#pragma unroll
                for (int n = 0; n < NT_O; ++n) {
                    o_acc[n][2 * rs] *= alpha;
                    o_acc[n][2 * rs + 1] *= alpha;
                }
            }
            if (!G16) {
#pragma unroll
                for (int kt = 0; kt < TOK / 16; ++kt) pa[kt][1] = pa[kt][3] = 0u;
            }

            // ---- O += P.V
#pragma unroll
            for (int kt = 0; kt < TOK / 16; ++kt) {
                const uint32_t tok = kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int np = 0; np < NT_O / 2; ++np) {
                    const uint32_t chunk = np * 2 + (lane >> 4);
                    const uint32_t addr = sV + (chunk >> 3) * (TOK * 128) + tok * 128 + (((chunk & 7) ^ (tok & 7)) << 4);
                    uint32_t b[4];
                    ldsm_x4_trans(addr, b);
                    mma_16816(o_acc[2 * np], pa[kt], b[0], b[1]);
                    mma_16816(o_acc[2 * np + 1], pa[kt], b[2], b[3]);
                }
            }
            __syncwarp();
            if (j + stages < n_tiles) issue(j + stages);
        }
        if (dead) break;

        // ---- end of piece: row sums over the quad
#pragma unroll
        for (int rs = 0; rs < ROWSETS; ++rs) {
            l_run[rs] += __shfl_xor_sync(0xffffffffu, l_run[rs], 1);
            l_run[rs] += __shfl_xor_sync(0xffffffffu, l_run[rs], 2);
        }

        if (n_parts > 1) {
            // un-normalised partial -> workspace, fragment order (coalesced)
            const size_t unit = static_cast<size_t>(part_slot) * kDecodeWarps + warp;
            if (G16) {
                float4* wo = reinterpret_cast<float4*>(prm.work_o) + unit * NT_O * 32;
#pragma unroll
                for (int n = 0; n < NT_O; ++n)
                    wo[n * 32 + lane] = make_float4(o_acc[n][0], o_acc[n][1], o_acc[n][2], o_acc[n][3]);
                reinterpret_cast<float4*>(prm.work_ml)[unit * 32 + lane] =
                    make_float4(m_run[0], l_run[0], m_run[1], l_run[1]);
            } else {
                float2* wo = reinterpret_cast<float2*>(prm.work_o) + unit * NT_O * 32;
#pragma unroll
                for (int n = 0; n < NT_O; ++n) wo[n * 32 + lane] = make_float2(o_acc[n][0], o_acc[n][1]);
                reinterpret_cast<float2*>(prm.work_ml)[unit * 32 + lane] = make_float2(m_run[0], l_run[0]);
            }
            __threadfence();
            __syncwarp();
            uint32_t old = 0;
            if (lane == 0) old = atomicAdd(prm.counters + seg * kDecodeWarps + warp, 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old != n_parts - 1) continue;  // someone else will merge
            __threadfence();
            // ---- last arrival: merge all partials of (request, head)
            float mstar[2] = {-INFINITY, -INFINITY};
            for (uint32_t k = 0; k < n_parts; ++k) {
                const size_t u = static_cast<size_t>(seg_first_slot + k) * kDecodeWarps + warp;
                if (G16) {
                    const float4 ml = ld_cg_f4(reinterpret_cast<const float4*>(prm.work_ml) + u * 32 + lane);
                    mstar[0] = fmaxf(mstar[0], ml.x);
                    mstar[1] = fmaxf(mstar[1], ml.z);
                } else {
                    const float2 ml = ld_cg_f2(reinterpret_cast<const float2*>(prm.work_ml) + u * 32 + lane);
                    mstar[0] = fmaxf(mstar[0], ml.x);
                }
            }
#pragma unroll
            for (int n = 0; n < NT_O; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
            l_run[0] = l_run[1] = 0.f;
            for (uint32_t k = 0; k < n_parts; ++k) {
                const size_t u = static_cast<size_t>(seg_first_slot + k) * kDecodeWarps + warp;
                if (G16) {
                    const float4 ml = ld_cg_f4(reinterpret_cast<const float4*>(prm.work_ml) + u * 32 + lane);
                    const float w0 = ex2(ml.x - mstar[0]), w1 = ex2(ml.z - mstar[1]);
                    l_run[0] += ml.y * w0;
                    l_run[1] += ml.w * w1;
                    const float4* wo = reinterpret_cast<const float4*>(prm.work_o) + u * NT_O * 32;
#pragma unroll
                    for (int n = 0; n < NT_O; ++n) {
                        const float4 v = ld_cg_f4(wo + n * 32 + lane);
                        o_acc[n][0] += v.x * w0; o_acc[n][1] += v.y * w0;
                        o_acc[n][2] += v.z * w1; o_acc[n][3] += v.w * w1;
                    }
                } else {
                    const float2 ml = ld_cg_f2(reinterpret_cast<const float2*>(prm.work_ml) + u * 32 + lane);
                    const float w0 = ex2(ml.x - mstar[0]);
                    l_run[0] += ml.y * w0;
                    const float2* wo = reinterpret_cast<const float2*>(prm.work_o) + u * NT_O * 32;
#pragma unroll
                    for (int n = 0; n < NT_O; ++n) {
                        const float2 v = ld_cg_f2(wo + n * 32 + lane);
                        o_acc[n][0] += v.x * w0; o_acc[n][1] += v.y * w0;
                    }
                }
            }
            m_run[0] = mstar[0];
            m_run[1] = mstar[1];
            if (lane == 0) prm.counters[seg * kDecodeWarps + warp] = 0u;  // ready for the next launch
        }

        // ---- write the rows of this (request, KV head)
#pragma unroll
        for (int rs = 0; rs < ROWSETS; ++rs) {
            const uint32_t row = qrow + 8 * rs;
            if (row >= prm.G) continue;
            const size_t hrow = static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G + row;
            if (prm.o_partial) {
                float* dst = prm.o_partial + hrow * D;
#pragma unroll
                for (int n = 0; n < NT_O; ++n)
                    *reinterpret_cast<float2*>(dst + n * 8 + qcol) = make_float2(o_acc[n][2 * rs], o_acc[n][2 * rs + 1]);
                if ((lane & 3) == 0) {
                    // natural-log units for the caller: m_nat = m_2 * ln 2
                    prm.ml_partial[hrow * 2] = m_run[rs] * 0.6931471805599453f;
                    prm.ml_partial[hrow * 2 + 1] = l_run[rs];
                }
            } else {
                const float inv = l_run[rs] > 0.f ? 1.0f / l_run[rs] : 0.f;
                if (prm.o_f32) {
                    float* dst = static_cast<float*>(prm.o) + hrow * D;
#pragma unroll
                    for (int n = 0; n < NT_O; ++n)
                        *reinterpret_cast<float2*>(dst + n * 8 + qcol) =
                            make_float2(o_acc[n][2 * rs] * inv, o_acc[n][2 * rs + 1] * inv);
                } else {
                    __half* dst = static_cast<__half*>(prm.o) + hrow * D;
#pragma unroll
                    for (int n = 0; n < NT_O; ++n)
                        *reinterpret_cast<__half2*>(dst + n * 8 + qcol) =
                            __floats2half2_rn(o_acc[n][2 * rs] * inv, o_acc[n][2 * rs + 1] * inv);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------
static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

bool decode_tma_shape_supported(size_t H, size_t KVH, size_t D, size_t P, size_t capacity) {
    if (D != 64 && D != 128) return false;
    if (P % kTileTokens != 0 || P / kTileTokens > 8) return false;
    if (KVH == 0 || H / KVH > 16) return false;
    if ((KVH + kDecodeWarps - 1) / kDecodeWarps > 16) return false;
    if (capacity == 0 || capacity > (size_t(1) << 25)) return false;
    return true;
}

bool decode_tma_pointers_supported(const AttnArgs& a) {
    if (!aligned(a.k_pages, 16) || !aligned(a.v_pages, 16)) return false;
    if (!aligned(a.q, a.q_dtype == MLC_F32 ? 8 : 4)) return false;
    if (a.o && !aligned(a.o, a.o_dtype == MLC_F32 ? 8 : 4)) return false;
    if (a.o_partial && (!aligned(a.o_partial, 8) || !a.ml_partial)) return false;
    return true;
}

template <int D, bool G16>
static int launch_t(mlc_ctx* ctx, const AttnArgs& a, const DecodePlanView& plan, const DecodeParams& prm,
                    const CUtensorMap* mk, const CUtensorMap* mv, uint32_t stages) {
    const size_t smem = static_cast<size_t>(kDecodeWarps) * stages * (2 * kTileTokens * D * 2) + 1024;
    size_t& configured = ctx->decode_smem_set[(D == 128 ? 2 : 0) + (G16 ? 1 : 0)];
    if (smem > configured) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(paged_decode_tma_kernel<D, G16>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured = smem;
    }
    (void)a;
    paged_decode_tma_kernel<D, G16><<<plan.n_cta, kDecodeWarps * 32, smem, ctx->stream>>>(*mk, *mv, prm);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

int launch_attention_decode_tma(mlc_ctx* ctx, const AttnArgs& a, const DecodePlanView& plan) {
    const uint32_t G = static_cast<uint32_t>(a.H / a.KVH);
    const bool g16 = G > 8;
    const size_t frag_floats = (g16 ? 4 : 2) * 32 * (a.D / 8);  // per (slot, warp)
    const size_t ml_floats = (g16 ? 4 : 2) * 32;
    const size_t units = static_cast<size_t>(plan.n_slots) * kDecodeWarps;
    const size_t o_bytes = units * frag_floats * 4, ml_bytes = units * ml_floats * 4;
    int st = ensure_workspace(ctx, o_bytes + ml_bytes + 256, static_cast<size_t>(plan.n_segs) * kDecodeWarps + 1);
    if (st != MLC_OK) return st;
    const CUtensorMap *mk = nullptr, *mv = nullptr;
    if ((st = get_tensor_map(ctx, a.k_pages, a, &mk)) != MLC_OK) return st;
    CUtensorMap mk_copy = *mk;  // the cache may grow while the second map is made
    if ((st = get_tensor_map(ctx, a.v_pages, a, &mv)) != MLC_OK) return st;

    DecodeParams prm{};
    prm.q = a.q;
    prm.o = a.o;
    prm.o_partial = a.o_partial;
    prm.ml_partial = a.ml_partial;
    prm.cta_counts = plan.cta_counts;
    prm.pieces = plan.pieces;
    prm.tile_pages = plan.tile_pages;
    prm.zero_rows = plan.zero_rows;
    prm.work_o = static_cast<float*>(ctx->d_work);
    prm.work_ml = reinterpret_cast<float*>(static_cast<char*>(ctx->d_work) + ((o_bytes + 255) / 256) * 256);
    prm.counters = ctx->d_counters;
    prm.err = ctx->d_err;
    prm.max_pieces = plan.max_pieces;
    prm.max_tiles = plan.max_tiles;
    prm.n_zero = plan.n_zero;
    prm.H = static_cast<uint32_t>(a.H);
    prm.KVH = static_cast<uint32_t>(a.KVH);
    prm.G = G;
    prm.sub_per_page = static_cast<uint32_t>(a.P / kTileTokens);
    prm.scale_log2 = a.scale * 1.4426950408889634f;
    prm.q_f32 = a.q_dtype == MLC_F32;
    prm.o_f32 = a.o_dtype == MLC_F32;
    const char* env = std::getenv("MLC_B200_DECODE_STAGES");
    uint32_t stages = env && *env ? static_cast<uint32_t>(std::atoi(env)) : 3u;
    if (stages < 1) stages = 1;
    if (stages > 8) stages = 8;
    prm.stages = stages;
    if (a.D == 64) return g16 ? launch_t<64, true>(ctx, a, plan, prm, &mk_copy, mv, stages)
                              : launch_t<64, false>(ctx, a, plan, prm, &mk_copy, mv, stages);
    return g16 ? launch_t<128, true>(ctx, a, plan, prm, &mk_copy, mv, stages)
               : launch_t<128, false>(ctx, a, plan, prm, &mk_copy, mv, stages);
}

}  // namespace mlcb
