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
// The four warps of a CTA work on the four KV heads of one head block over the same
// tiles, so together they read whole token rows (KVH*D contiguous halfs) of a page at
// about the same time. That matters: fetching one head's 128-byte slices alone
// (512-byte stride) was measured at roughly half the DRAM throughput of the dense
// pattern on B200.
//
// G = 8 means 4 FMA per KV byte; at HBM speed that is more than half of the
// SM's fp32 FMA rate before any fp16->fp32 conversion, so the dots go through the
// tensor cores and the kernel stays bandwidth-bound. tcgen05/TMEM is not used
// here: a decode tile has 8 (or 4) query rows against the 64-row minimum of a
// tcgen05 MMA, and the accumulators fit in registers.
//
// A (request, head block) that spans several CTAs leaves one un-normalised partial
// (o, m, l) per piece in a workspace - plain stores, no fence, no counter - and a
// second small kernel, chained to the first by programmatic dependent launch, merges
// them with the log-sum-exp rule and writes O. The kernel boundary is the only
// synchronisation between the two.
//
// Decode-step variant (`step` launches): the kernel also writes the step's new K/V
// row of every request into the pool - the reference's two
// scatter_kv_paged_batched_f16 dispatches (metal_runtime.mm:405-424) - and uses the
// row from its source buffer, so no separate scatter launch has to finish first. It is
// launched with programmatic stream serialisation: everything that depends only on
// the plan and on K/V rows written by earlier steps (plan reads, barrier set-up, the
// first ring-full of TMA copies) runs before griddepcontrol.wait, i.e. while the
// previous kernels in the stream are still draining; Q and the new rows are read
// after it.
//
// Nothing here spins on another CTA. The only waits are mbarrier waits on this
// warp's own TMA copies; they are bounded, and on expiry the warp records
// MLC_DEVERR_WAIT_TIMEOUT and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <vector>

#include "attn_internal.hpp"

namespace mlcb {

// ------------------------------------------------------------------------------
// tensor maps
// ------------------------------------------------------------------------------
struct TensorMapCache {
    struct Entry {
        const void* pool;
        const void* pool2;   // second pool of a K/V pair map, else null
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
// Encodes the map for one pool; pure host arithmetic inside the driver, no allocation.
static int encode_tensor_map(mlc_ctx* ctx, const void* pool, const AttnArgs& a, CUtensorMap* out) {
    if (!ctx->tmap_encode_fn) {
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->tmap_encode_fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !ctx->tmap_encode_fn)
            return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    cuuint64_t dims[4] = {a.D, a.KVH, a.P, a.capacity};
    cuuint64_t strides[3] = {a.D * 2, a.KVH * a.D * 2, a.P * a.KVH * a.D * 2};
    cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(kTileTokens), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode_fn)(
        out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(pool), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return MLC_OK;
}

// One map over both pools of a layer: a fifth dimension of extent 2 whose stride is the distance between
// the pools, so that one TMA instruction fetches the K tile and the V tile of a stage (a TMA instruction
// costs the issuing lane 75-95 clocks, measured). The lower pool is index 0. Possible when the pools do
// not coincide and their distance is a multiple of 16 bytes below 2^40 (the tensor-map stride rules).
static bool pair_map_possible(const void* k_pool, const void* v_pool) {
    const uintptr_t k = reinterpret_cast<uintptr_t>(k_pool), v = reinterpret_cast<uintptr_t>(v_pool);
    const uintptr_t dist = k < v ? v - k : k - v;
    return dist != 0 && dist % 16 == 0 && dist < (uintptr_t(1) << 40);
}
static int encode_pair_map(mlc_ctx* ctx, const void* k_pool, const void* v_pool, const AttnArgs& a, CUtensorMap* out) {
    if (!ctx->tmap_encode_fn) {
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->tmap_encode_fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !ctx->tmap_encode_fn)
            return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    const uintptr_t k = reinterpret_cast<uintptr_t>(k_pool), v = reinterpret_cast<uintptr_t>(v_pool);
    cuuint64_t dims[5] = {a.D, a.KVH, a.P, a.capacity, 2};
    cuuint64_t strides[4] = {a.D * 2, a.KVH * a.D * 2, a.P * a.KVH * a.D * 2, k < v ? v - k : k - v};
    cuuint32_t box[5] = {64, 1, static_cast<cuuint32_t>(kTileTokens), 1, 2};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode_fn)(
        out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, reinterpret_cast<void*>(k < v ? k : v), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled (K/V pair) failed (%d)", static_cast<int>(r));
    return MLC_OK;
}

static int get_tensor_map(mlc_ctx* ctx, const void* pool, const AttnArgs& a, CUtensorMap* out, const void* pool2 = nullptr) {
    if (!ctx->tmap_cache) ctx->tmap_cache = new TensorMapCache();
    TensorMapCache& tc = *ctx->tmap_cache;
    for (auto& e : tc.entries)
        if (e.pool == pool && e.pool2 == pool2 && e.D == a.D && e.KVH == a.KVH && e.P == a.P && e.capacity == a.capacity) {
            *out = e.map;
            return MLC_OK;
        }
    TensorMapCache::Entry e{pool, pool2, a.D, a.KVH, a.P, a.capacity, {}};
    int st = pool2 ? encode_pair_map(ctx, pool, pool2, a, &e.map) : encode_tensor_map(ctx, pool, a, &e.map);
    if (st != MLC_OK) return st;
    if (tc.entries.size() >= 256) tc.entries.erase(tc.entries.begin());
    tc.entries.push_back(e);
    *out = e.map;
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
    const SegDesc* seg_desc;
    float* work_o;      // split-KV workspace: o fragments
    float* work_ml;     // split-KV workspace: (m, l) per lane
    uint32_t* err;
    // decode-step variant: the step's new rows (fp16 [batch, KVH, D]) and the pools they go to
    const __half* k_new;
    const __half* v_new;
    __half* k_pool;
    __half* v_pool;
    uint32_t max_pieces, max_tiles, n_zero;
    uint32_t H, KVH, G, P;
    uint32_t stages;
    float scale_log2;   // scale * log2(e)
    int q_f32, o_f32;
    int step;           // 1: decode-step variant (fused row write, early start)
    int pdl;            // 1: launched with programmatic stream serialisation
    int early_fetch;    // 1: a decode step may fetch tiles of earlier steps' rows before griddepcontrol.wait
    int fresh_rows;     // 1: not a decode step, but the kernel in front wrote only the rows the plan marks as fresh
    unsigned long long* trace;  // optional [cta][warp][8] %globaltimer stamps (MLC_B200_TRACE)
    // In-kernel merge: one arrival counter per (split segment, warp); null = a merge kernel follows.
    uint32_t* seg_counters;
    uint32_t n_segs;
    // head_dim 64: the first tensor map covers both pools (one TMA instruction per stage); k_off / v_off are
    // the tiles' byte offsets inside a stage (the lower pool comes first)
    uint32_t kv_pair, k_off, v_off;
    // whole-pass launch: layers of the pass, and the CTAs the (single-layer) plan was made for
    uint32_t n_layers, plan_ctas;
    // unit mode: KV heads a CTA works on at a time (1: the W warps share one (request, head); h > 1: warp w
    // holds head w % h of the item's head group and part w / h of that head's tiles, so that the CTA's
    // warps fetch h adjacent 128-byte chunks of every token row at about the same time)
    uint32_t hpc;
    // whole-pass launch: bytes of the Q block and of the O block of one work item (the hpc * G query heads of a
    // request's head group are adjacent rows), staged through shared memory so that both cross the memory
    // system - or the PCIe link, when the caller's buffers are host memory - in whole 16-byte-per-thread rows
    uint32_t q_block_bytes, o_block_bytes;
};

// One layer of a whole-pass launch: what differs between the layers of a decode pass.
struct alignas(64) LayerArgs {
    CUtensorMap map_k;   // the K/V pair map at head_dim 64 when the pools allow it, else the K pool's
    CUtensorMap map_v;
    const void* q;
    void* o;
    const __half* k_new;
    const __half* v_new;
    __half* k_pool;
    __half* v_pool;
    uint32_t kv_pair, k_off, v_off, pad;
};
static constexpr int kMaxPassLayers = 64;
// All layers of a pass as ONE kernel parameter (20 KiB; kernel parameters may be up to 32764 bytes), so that
// the launch needs no staging copy and is captured whole by a CUDA graph.
struct PassArgs {
    LayerArgs layer[kMaxPassLayers];
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
// Bounded wait: a poll that finds the phase open suspends for a few microseconds (measured ~4 us),
// so 2^18 polls are about a second before giving up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    {  // non-blocking test first: a phase that has already completed is the common case (measured ~0.5 % per layer)
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    for (uint32_t i = 0; i < (1u << 18); ++i)
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
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// Same with a compile-time byte offset folded into the address operand.
template <int OFF>
__device__ __forceinline__ void ldsm_x4_off(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ void ldsm_x4_trans_off(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(OFF));
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

// Writes the rows of one (request, KV head) from accumulator fragments: either O
// (normalised, fp32 or fp16) or the caller-visible partial (un-normalised o, (m, l)).
template <int D, bool G16>
__device__ __forceinline__ void write_rows(const DecodeParams& prm, uint32_t req, uint32_t head, uint32_t lane,
                                           const float (&o_acc)[D / 8][4], const float (&m_run)[2],
                                           const float (&l_run)[2]) {
    constexpr int NT_O = D / 8;
    constexpr int ROWSETS = G16 ? 2 : 1;
    const uint32_t qrow = lane >> 2, qcol = (lane & 3) * 2;
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

// ------------------------------------------------------------------------------
// the attention kernel
// ------------------------------------------------------------------------------
template <int D, bool G16, bool CG>
__device__ __forceinline__ void merge_segment(const DecodeParams& prm, const SegDesc& sd, uint32_t warp, uint32_t lane);

// Split-KV across GPUs, fused into the attention kernel (PEER instantiation of the body below): what a
// rank needs to hand the finished rows of a (request, head) to every rank and to combine all ranks' rows.
struct PeerParams {
    char* peer[16];          // gather buffers of all ranks as mapped into this process (own one included)
    char* local;             // this rank's own gather buffer
    void* out;               // final O [rows, D] on this rank
    uint32_t* seq;           // step counter (local; advanced by the last CTA of a launch to finish)
    uint32_t* done;          // CTAs of this launch that have finished
    size_t ll_off;           // byte offset of the stamped slots [2 parities][world]
    size_t ll_slot_bytes;    // bytes of one slot: max_rows * (D * 8 + 16)
    uint32_t rank, world, max_rows, max_polls, out_f32;
};

// The kernel of the per-layer entry points. It is the same algorithm as decode_body below with a single item
// per CTA (no layers to walk, one KV head per CTA item) and is kept as a body of its own on purpose: the tile
// loop of this kernel runs at about a quarter of an instruction per clock on one warp per scheduler, and the
// register allocation the compiler finds for it moves its time per layer by several per cent when code is
// added around the loop (measured: 8.37 us per layer for this body, 8.6 - 8.9 us for the generalised one at
// the same work), so the generalised body is used where it is needed - the whole-pass launch - only.
// UNIT = false: the four warps of a CTA are the four KV heads of a head block over the same tiles
// (dense 512-byte rows), requests are cut over CTAs and split requests merged afterwards.
// UNIT = true ("unit mode", the planner's choice unless one request dwarfs the others): no request
// is split over CTAs. Every warp has its own piece and tile lists; the W warps of a CTA (8 for
// head_dim 64, 4 for 128) take the W parts of one (request, head) at a time and merge through
// shared memory, so there are no global partials and no merge kernel. More warps matter: a warp
// needs ~0.8 us per 32-token tile (dependent mma.sync / ldmatrix / shuffle chains, one warp per
// scheduler), so the longest unit's time falls with the number of warps that share it.
// PEER (unit mode): the rank holds a slice of every request's pages. The CTA that finishes a (request, head)
// - the only one that worked on it, or the last of the CTAs it was cut over - stores the un-normalised rows
// (o, m, l) straight into every rank's gather buffer over NVLink peer memory (plain 16-byte stores, no loads
// from a peer, no TMA, no multicast). Every float travels beside the step's stamp in one 8-byte unit
// {value, stamp} (two per store), so a reader knows from the bytes themselves that a value is this step's:
// no flag behind a system-scope fence, whose round trips cost more than the 33 KiB of rows do. The same CTA
// then reads every rank's rows of that (request, head) from its OWN memory, polling - bounded - the units
// whose stamp is not there yet, combines them with the log-sum-exp rule and writes O. One launch per step.
template <int D, bool G16, bool UNIT, bool PEER>
__device__ __forceinline__ void decode_layer_body(const CUtensorMap& tmK, const CUtensorMap& tmV, const DecodeParams& prm,
                                                  const PeerParams* pp) {
    constexpr int TOK = kTileTokens;
    constexpr int NT_S = TOK / 8;          // score n-tiles per tile
    constexpr int KSTEPS = D / 16;         // k-steps of Q.K^T
    constexpr int NT_O = D / 8;            // output n-tiles
    constexpr int SUBS = D / 64;           // 64-half boxes per row
    constexpr uint32_t kTileBytes = TOK * D * 2;       // one of K or V
    constexpr uint32_t kStageBytes = 2 * kTileBytes;
    constexpr int ROWSETS = G16 ? 2 : 1;
    constexpr int W = UNIT ? unit_warps(D) : kDecodeWarps;  // warps of this CTA

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[W][8];
    __shared__ uint32_t last_part_flag;  // unit mode: this CTA brought the last piece of a (request, head) cut over CTAs

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = blockIdx.x;
    const uint32_t stages = prm.stages;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring = smem_base + warp * stages * kStageBytes;

    // The three plan reads of the prologue are independent of one another, so they
    // cost one memory round trip together: the CTA's counts, its first 32 tile words
    // (one per lane) and its first 16 piece descriptors (half a descriptor per lane).
    // The planner pads both arrays so that these reads stay inside the plan image.
    const uint32_t vcta = UNIT ? cta * W + warp : cta;  // unit mode: one plan slice per warp
    const uint32_t* my_tiles = prm.tile_pages + static_cast<size_t>(vcta) * prm.max_tiles;
    const PieceDesc* my_pieces = prm.pieces + static_cast<size_t>(vcta) * prm.max_pieces;
    const uint2 counts = __ldg(reinterpret_cast<const uint2*>(prm.cta_counts) + vcta);
    uint32_t win_base = 0;
    uint32_t win = __ldg(my_tiles + lane);
    const uint4 desc_half = __ldg(reinterpret_cast<const uint4*>(my_pieces) + lane);
    const uint32_t n_pieces = counts.x, n_tiles = counts.y;
    auto stamp = [&](int i) {
        if (prm.trace && lane == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            prm.trace[(static_cast<size_t>(cta) * W + warp) * 8 + i] = t;
        }
    };
    stamp(0);

    if (lane == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(smem_u32(&bars[warp][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    auto tile_entry = [&](uint32_t j) -> uint32_t {
        if (j - win_base >= 32u) {  // uniform across the warp
            win_base = j & ~31u;
            win = (win_base + lane < n_tiles) ? __ldg(my_tiles + win_base + lane) : 0u;
        }
        return __shfl_sync(0xffffffffu, win, j - win_base);
    };
    // Ring position counters of this warp. They count only tiles of head blocks in
    // which this warp owns a KV head, in the (identical) order of issue and use.
    // (kept as wrapping stage indices and a parity bit: the ring depth is a run-time value, and a
    // division by it per tile costs tens of instructions)
    uint32_t iss_stage = 0, con_stage = 0, con_parity = 0;
    // Issues the TMA copies of the tile word `e` into the next ring stage.
    auto issue_word = [&](uint32_t e) {
        const uint32_t hfield = (e >> kTileHbShift) & kTileHbMask;   // head block, or the head itself in unit mode
        const uint32_t head = UNIT ? hfield : hfield * kDecodeWarps + warp;
        if (!UNIT && head >= prm.KVH) return;  // this warp has no KV head in that head block
        const uint32_t s = iss_stage;
        iss_stage = (iss_stage + 1 == stages) ? 0u : iss_stage + 1;
        if (lane == 0) {
            const uint32_t bar = smem_u32(&bars[warp][s]);
            const uint32_t dst = ring + s * kStageBytes;
            const int page = static_cast<int>(e & kTilePageMask);
            const int slot0 = static_cast<int>(((e >> kTileSubShift) & 7u) * TOK);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, kStageBytes);
            if (D == 64 && prm.kv_pair) {
                tma_load_5d(dst, &tmK, bar, 0, static_cast<int>(head), slot0, page, 0);
            } else {
#pragma unroll
                for (int sub = 0; sub < SUBS; ++sub) {
                    tma_load_4d(dst + sub * (TOK * 128), &tmK, bar, sub * 64, static_cast<int>(head), slot0, page);
                    tma_load_4d(dst + kTileBytes + sub * (TOK * 128), &tmV, bar, sub * 64, static_cast<int>(head), slot0, page);
                }
            }
        }
    };

    // Prefetches run ahead over piece boundaries; they need nothing but the tile list.
    // In a decode step, tiles that hold a row written in this step ("fresh" tiles: the
    // ones containing the new token) are not fetched before griddepcontrol.wait;
    // everything older may be.
    uint32_t next_issue = 0;  // next CTA-local tile to fetch
    const uint32_t window = n_tiles < stages ? n_tiles : stages;
    if (prm.pdl) {
        if ((prm.step || prm.fresh_rows) && prm.early_fetch) {
            while (next_issue < window) {
                const uint32_t e = tile_entry(next_issue);
                if (e & kTileFreshBit) break;
                issue_word(e);
                ++next_issue;
            }
        }
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    while (next_issue < window) {
        issue_word(tile_entry(next_issue));
        ++next_issue;
    }
    stamp(1);
    // PEER: the step number (read after the launch before this one has completed: its last CTA advances it),
    // the slots this rank writes in every rank's buffer and the flags it sets and waits for
    uint32_t peer_step = 0;
    if constexpr (PEER) peer_step = *reinterpret_cast<volatile uint32_t*>(pp->seq);
    const uint32_t peer_parity = peer_step & 1u, peer_stamp = peer_step + 1u;   // never 0: zeroed flags match nothing
    auto peer_slot = [&](uint32_t r) -> char* {    // this rank's stamped slot in rank r's buffer
        return pp->peer[r] + pp->ll_off + (static_cast<size_t>(peer_parity) * pp->world + pp->rank) * pp->ll_slot_bytes;
    };
    // two values of row `hrow`, columns col / col + 1 (col even), to every rank
    auto peer_store_o = [&](size_t hrow, uint32_t col, float a, float b) {
        const uint4 v = make_uint4(__float_as_uint(a), peer_stamp, __float_as_uint(b), peer_stamp);
        for (uint32_t k = 0; k < pp->world; ++k)
            *reinterpret_cast<uint4*>(peer_slot(k) + (hrow * D + col) * 8) = v;
    };
    auto peer_store_ml = [&](size_t hrow, float m_nat, float l) {
        const uint4 v = make_uint4(__float_as_uint(m_nat), peer_stamp, __float_as_uint(l), peer_stamp);
        for (uint32_t k = 0; k < pp->world; ++k)
            *reinterpret_cast<uint4*>(peer_slot(k) + static_cast<size_t>(pp->max_rows) * D * 8 + hrow * 16) = v;
    };
    // Reads a stamped 16-byte unit of this rank's own memory, again and again until both halves carry this
    // step's stamp; false when the limit runs out.
    auto peer_wait = [&](const char* addr, float& a, float& b) -> bool {
        for (uint32_t i = 0; i < pp->max_polls; ++i) {
            uint4 v;
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
            if (v.y == peer_stamp && v.w == peer_stamp) {
                a = __uint_as_float(v.x);
                b = __uint_as_float(v.z);
                return true;
            }
        }
        return false;
    };
    // Rows [row0, row0 + G) of a (request, head) this CTA has just stored to every rank: combine what every
    // rank stored here. m* = max_k m_k, w_k = exp(m_k - m*), O = sum_k o_k w_k / sum_k l_k w_k.
    auto peer_finish = [&](size_t row0) {
        if constexpr (PEER) {
            const char* base = pp->local + pp->ll_off + static_cast<size_t>(peer_parity) * pp->world * pp->ll_slot_bytes;
            for (uint32_t t = threadIdx.x; t < prm.G * (D / 2); t += blockDim.x) {
                const size_t row = row0 + t / (D / 2);
                const uint32_t col = (t % (D / 2)) * 2;
                float m[16], l[16], mstar = -INFINITY;
                bool ok = true;
                for (uint32_t k = 0; k < pp->world && ok; ++k) {
                    ok = peer_wait(base + k * pp->ll_slot_bytes + static_cast<size_t>(pp->max_rows) * D * 8 + row * 16, m[k], l[k]);
                    mstar = fmaxf(mstar, m[k]);
                }
                float lsum = 0.f, a0 = 0.f, a1 = 0.f;
                for (uint32_t k = 0; k < pp->world && ok; ++k) {
                    float x, y;
                    ok = peer_wait(base + k * pp->ll_slot_bytes + (row * D + col) * 8, x, y);
                    const float w = (m[k] == -INFINITY) ? 0.f : expf(m[k] - mstar);
                    lsum += l[k] * w;
                    a0 += x * w;
                    a1 += y * w;
                }
                if (!ok) {    // a rank's rows did not arrive in time: no output for this row, the context stays usable
                    atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT | (0x51u << 8));
                    continue;
                }
                const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
                if (pp->out_f32) *reinterpret_cast<float2*>(static_cast<float*>(pp->out) + row * D + col) = make_float2(a0 * inv, a1 * inv);
                else *reinterpret_cast<__half2*>(static_cast<__half*>(pp->out) + row * D + col) = __floats2half2_rn(a0 * inv, a1 * inv);
            }
        }
    };

    // Requests that attend to nothing: their O rows are zeros (mm:2254-2257).
    for (uint32_t i = cta; i < prm.n_zero; i += gridDim.x) {
        const uint32_t r = prm.zero_rows[i];
        if constexpr (PEER) {
            // this rank holds no token of the request: its rows weigh nothing, but the other ranks wait for them
            for (uint32_t e = threadIdx.x; e < prm.H * (D / 2); e += blockDim.x)
                peer_store_o(static_cast<size_t>(r) * prm.H + e / (D / 2), (e % (D / 2)) * 2, 0.f, 0.f);
            for (uint32_t e = threadIdx.x; e < prm.H; e += blockDim.x) peer_store_ml(static_cast<size_t>(r) * prm.H + e, -INFINITY, 0.f);
            for (uint32_t h = 0; h < prm.KVH; ++h) peer_finish(static_cast<size_t>(r) * prm.H + static_cast<size_t>(h) * prm.G);
            continue;
        }
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

    const uint32_t qrow = lane >> 2, qcol = (lane & 3) * 2;
    // Per-lane byte offsets of the ldmatrix rows inside a swizzled tile, computed once: a K fragment of
    // score tile n, k-pair kp sits at koff[kp] + n * 1024, a V fragment of token block kt, column pair np
    // at voff[np] + kt * 2048 (the token index only enters through lane & 7 and a multiple of 8 rows).
    // Kept in registers at head_dim 64 (6 values); at 128 the kernel has none to spare and recomputes them.
    constexpr bool kKeepOffsets = (D == 64);
    auto k_offset = [&](int kp) -> uint32_t {
        const uint32_t chunk = kp * 4 + (lane >> 3);
        return (chunk >> 3) * (TOK * 128) + (lane & 7) * 128 + (((chunk & 7) ^ (lane & 7)) << 4);
    };
    auto v_offset = [&](int np) -> uint32_t {
        const uint32_t chunk = np * 2 + (lane >> 4);
        return (chunk >> 3) * (TOK * 128) + ((lane & 7) + ((lane >> 3) & 1) * 8) * 128 + (((chunk & 7) ^ (lane & 7)) << 4);
    };
    uint32_t koff[kKeepOffsets ? KSTEPS / 2 : 1], voff[kKeepOffsets ? NT_O / 2 : 1];
    if constexpr (kKeepOffsets) {
#pragma unroll
        for (int kp = 0; kp < KSTEPS / 2; ++kp) koff[kp] = k_offset(kp);
#pragma unroll
        for (int np = 0; np < NT_O / 2; ++np) voff[np] = v_offset(np);
    }
    uint32_t j = 0;  // CTA-local tile counter (consume side)
    bool dead = false;

    uint32_t pi = 0;
    for (; pi < n_pieces && !dead; ++pi) {
        uint4 d0, d1;
        if (pi < 16u) {  // prefetched in the prologue: lane 2i holds the first half of piece i
            d0.x = __shfl_sync(0xffffffffu, desc_half.x, 2 * pi);
            d0.y = __shfl_sync(0xffffffffu, desc_half.y, 2 * pi);
            d0.z = __shfl_sync(0xffffffffu, desc_half.z, 2 * pi);
            d0.w = __shfl_sync(0xffffffffu, desc_half.w, 2 * pi);
            d1.x = __shfl_sync(0xffffffffu, desc_half.x, 2 * pi + 1);
            d1.y = __shfl_sync(0xffffffffu, desc_half.y, 2 * pi + 1);
            d1.z = __shfl_sync(0xffffffffu, desc_half.z, 2 * pi + 1);
            d1.w = __shfl_sync(0xffffffffu, desc_half.w, 2 * pi + 1);
        } else {
            d0 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi));
            d1 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi) + 1);
        }
        const uint32_t req = d0.x, piece_tiles = d0.z, part_slot = d0.w;
        const uint32_t n_parts = d1.z & 0xffffu, hb = d1.z >> 16;
        const uint32_t last_valid = d1.w & 0xffffu;
        const bool fresh_piece = prm.step && ((d1.w >> 16) & 1u);  // its last tile holds the new token
        const uint32_t head = UNIT ? hb : hb * kDecodeWarps + warp;
        if (head >= prm.KVH) {  // keep the tile counter and the prefetch stream in step
            for (uint32_t t = 0; t < piece_tiles; ++t, ++j) {
                if (next_issue < n_tiles) {
                    issue_word(tile_entry(next_issue));
                    ++next_issue;
                }
            }
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
        // ---- decode step: this step's new K/V row of (request, head), one 16-byte chunk per
        // lane (lanes [0, D/8) hold K, lanes [16, 16 + D/8) hold V). It is written to the pool
        // here and patched over the fresh tile's copy in shared memory below.
        uint4 new_row = make_uint4(0u, 0u, 0u, 0u);
        constexpr uint32_t kRowChunks = D / 8;
        const bool row_lane = (lane & 15u) < kRowChunks;
        if (fresh_piece && row_lane) {
            const __half* src = (lane < 16u ? prm.k_new : prm.v_new) +
                                (static_cast<size_t>(req) * prm.KVH + head) * D + (lane & 15u) * 8;
            new_row = *reinterpret_cast<const uint4*>(src);
        }

        float o_acc[NT_O][4];
#pragma unroll
        for (int n = 0; n < NT_O; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        for (uint32_t t = 0; t < piece_tiles; ++t, ++j) {
            const uint32_t s = con_stage;
            const uint32_t bar = smem_u32(&bars[warp][s]);
            const uint32_t parity = con_parity;
            if (++con_stage == stages) {
                con_stage = 0;
                con_parity ^= 1u;
            }
            if (!mbar_wait_bounded(bar, parity)) {
                if (lane == 0) atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT);
                dead = true;
                break;
            }
            if (j == 0) stamp(2);
            // the next tile word to fetch, taken now so that its shuffle (and every 32nd time the load of
            // the next window) is long done when lane 0 needs it at the end of the tile
            const uint32_t e_next = next_issue < n_tiles ? tile_entry(next_issue) : 0u;
            const uint32_t sK = ring + s * kStageBytes + prm.k_off, sV = ring + s * kStageBytes + prm.v_off;
            const bool last_tile = t + 1 == piece_tiles;
            const uint32_t nv = last_tile ? last_valid : TOK;

            if (fresh_piece && last_tile) {
                // The new token is the last valid row of this tile; its pool address follows
                // from the tile word (page, sub-tile).
                const uint32_t rowi = nv - 1;
                const uint32_t e = __ldg(my_tiles + j);
                if (row_lane) {
                    const uint32_t chunk = lane & 15u;
                    const uint32_t addr = (lane < 16u ? sK : sV) + (chunk >> 3) * (TOK * 128) + rowi * 128 +
                                          (((chunk & 7) ^ (rowi & 7)) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(new_row.x), "r"(new_row.y),
                                 "r"(new_row.z), "r"(new_row.w) : "memory");
                    const size_t prow = (static_cast<size_t>(e & kTilePageMask) * prm.P +
                                         ((e >> kTileSubShift) & 7u) * TOK + rowi) * prm.KVH + head;
                    __half* dstp = (lane < 16u ? prm.k_pool : prm.v_pool) + prow * D + chunk * 8;
                    *reinterpret_cast<uint4*>(dstp) = new_row;
                }
                __syncwarp();
            }

            // ---- S = Q.K^T (fp32)
            // The shared-memory loads of a group of score tiles are all issued before the first MMA that
            // needs one (the asm statements keep their order, so load -> mma -> load -> mma would pay
            // the ldmatrix latency once per pair: ~1200 clocks per tile, measured), and the MMAs run
            // over independent accumulators in turn.
            float sc[NT_S][4];
            constexpr int kScoreGroup = (D == 64) ? NT_S : NT_S / 2;  // 32 fragment registers per group
#pragma unroll
            for (int n0 = 0; n0 < NT_S; n0 += kScoreGroup) {
                uint32_t kb[kScoreGroup][KSTEPS / 2][4];
#pragma unroll
                for (int kp = 0; kp < KSTEPS / 2; ++kp) {
                    const uint32_t addr = sK + (kKeepOffsets ? koff[kKeepOffsets ? kp : 0] : k_offset(kp)) + n0 * 1024;
                    static_assert(kScoreGroup <= 4, "unrolled by hand below");
                    ldsm_x4_off<0>(addr, kb[0][kp]);
                    if constexpr (kScoreGroup > 1) ldsm_x4_off<1024>(addr, kb[1][kp]);
                    if constexpr (kScoreGroup > 2) ldsm_x4_off<2048>(addr, kb[2][kp]);
                    if constexpr (kScoreGroup > 3) ldsm_x4_off<3072>(addr, kb[3][kp]);
                }
#pragma unroll
                for (int ni = 0; ni < kScoreGroup; ++ni) sc[n0 + ni][0] = sc[n0 + ni][1] = sc[n0 + ni][2] = sc[n0 + ni][3] = 0.f;
#pragma unroll
                for (int kp = 0; kp < KSTEPS / 2; ++kp) {
#pragma unroll
                    for (int ni = 0; ni < kScoreGroup; ++ni) mma_16816(sc[n0 + ni], qa[2 * kp], kb[ni][kp][0], kb[ni][kp][1]);
#pragma unroll
                    for (int ni = 0; ni < kScoreGroup; ++ni) mma_16816(sc[n0 + ni], qa[2 * kp + 1], kb[ni][kp][2], kb[ni][kp][3]);
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
                if (nv < TOK) {  // only a request's last tile is partly valid (warp-uniform)
#pragma unroll
                    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const uint32_t tok = n * 8 + qcol + e;
                            const float v = tok < nv ? sc[n][2 * rs + e] * prm.scale_log2 : -INFINITY;
                            sc[n][2 * rs + e] = v;
                            tmax = fmaxf(tmax, v);
                        }
                    }
                } else {
#pragma unroll
                    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float v = sc[n][2 * rs + e] * prm.scale_log2;
                            sc[n][2 * rs + e] = v;
                            tmax = fmaxf(tmax, v);
                        }
                    }
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run[rs], tmax);  // finite: every tile has >= 1 valid token
                float psum = 0.f;
#pragma unroll
                for (int n = 0; n < NT_S; ++n) {
                    const float p0 = ex2(sc[n][2 * rs] - m_new), p1 = ex2(sc[n][2 * rs + 1] - m_new);
                    psum += p0 + p1;
                    pa[n >> 1][rs + 2 * (n & 1)] = pack_half2(p0, p1);
                }
                // The accumulators are rescaled only when some row's maximum moved, which after the
                // first tiles of a request is rare (warp-uniform test).
                if (__any_sync(0xffffffffu, m_new > m_run[rs])) {
                    const float alpha = ex2(m_run[rs] - m_new);  // ex2(-inf) = 0 on the first tile
                    l_run[rs] *= alpha;
                    m_run[rs] = m_new;
#pragma unroll
                    for (int n = 0; n < NT_O; ++n) {
                        o_acc[n][2 * rs] *= alpha;
                        o_acc[n][2 * rs + 1] *= alpha;
                    }
                }
                l_run[rs] += psum;
            }
            if (!G16) {
#pragma unroll
                for (int kt = 0; kt < TOK / 16; ++kt) pa[kt][1] = pa[kt][3] = 0u;
            }

            // ---- O += P.V
            // same batching: the V fragments of 64 output columns first, then their MMAs
            constexpr int kOutGroup = 4;  // ldmatrix per batch = 16 fragment registers
#pragma unroll
            for (int kt = 0; kt < TOK / 16; ++kt) {
#pragma unroll
                for (int np0 = 0; np0 < NT_O / 2; np0 += kOutGroup) {
                    uint32_t vb[kOutGroup][4];
#pragma unroll
                    for (int i = 0; i < kOutGroup; ++i)
                        ldsm_x4_trans(sV + (kKeepOffsets ? voff[kKeepOffsets ? np0 + i : 0] : v_offset(np0 + i)) + kt * 2048, vb[i]);
#pragma unroll
                    for (int i = 0; i < kOutGroup; ++i) {
                        mma_16816(o_acc[2 * (np0 + i)], pa[kt], vb[i][0], vb[i][1]);
                        mma_16816(o_acc[2 * (np0 + i) + 1], pa[kt], vb[i][2], vb[i][3]);
                    }
                }
            }
            __syncwarp();
            if (next_issue < n_tiles) {
                issue_word(e_next);
                ++next_issue;
            }
        }
        if (dead) break;
        if (pi == 0) stamp(3);

        // ---- end of piece: row sums over the quad
#pragma unroll
        for (int rs = 0; rs < ROWSETS; ++rs) {
            l_run[rs] += __shfl_xor_sync(0xffffffffu, l_run[rs], 1);
            l_run[rs] += __shfl_xor_sync(0xffffffffu, l_run[rs], 2);
        }

        if (UNIT) {
            // The W warps hold the W parts of this (request, head): exchange the un-normalised
            // partials through shared memory, then every warp merges and writes its share of the
            // output columns.
            constexpr int FR = G16 ? 4 : 2;
            constexpr uint32_t kXWarpFloats = (NT_O + 1) * 32 * FR;
            float* xb = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) +
                        (static_cast<size_t>(W) * stages * kStageBytes) / 4;
            float* mine = xb + warp * kXWarpFloats;
#pragma unroll
            for (int n = 0; n < NT_O; ++n)
#pragma unroll
                for (int f = 0; f < FR; ++f) mine[(n * 32 + lane) * FR + f] = o_acc[n][f];
#pragma unroll
            for (int rs = 0; rs < ROWSETS; ++rs) {
                mine[(NT_O * 32 + lane) * FR + 2 * rs] = m_run[rs];
                mine[(NT_O * 32 + lane) * FR + 2 * rs + 1] = l_run[rs];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
            float wk[W][2], lstar[2], mstar[2];
#pragma unroll
            for (int rs = 0; rs < ROWSETS; ++rs) {
                float mk[W];
                mstar[rs] = -INFINITY;
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    mk[k] = xb[k * kXWarpFloats + (NT_O * 32 + lane) * FR + 2 * rs];
                    mstar[rs] = fmaxf(mstar[rs], mk[k]);
                }
                lstar[rs] = 0.f;
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    wk[k][rs] = (mk[k] == -INFINITY) ? 0.f : ex2(mk[k] - mstar[rs]);  // an empty quarter weighs nothing
                    lstar[rs] += xb[k * kXWarpFloats + (NT_O * 32 + lane) * FR + 2 * rs + 1] * wk[k][rs];
                }
            }
            // Writes rows of O (or of the caller's partial output) for output n-tile n.
            auto emit = [&](int n, const float (&acc)[FR], const float (&ls)[2]) {
#pragma unroll
                for (int rs = 0; rs < ROWSETS; ++rs) {
                    const uint32_t row = qrow + 8 * rs;
                    if (row >= prm.G) continue;
                    const size_t hrow = static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G + row;
                    if constexpr (PEER) {
                        peer_store_o(hrow, n * 8 + qcol, acc[2 * rs], acc[2 * rs + 1]);
                    } else if (prm.o_partial) {
                        *reinterpret_cast<float2*>(prm.o_partial + hrow * D + n * 8 + qcol) = make_float2(acc[2 * rs], acc[2 * rs + 1]);
                    } else {
                        const float inv = ls[rs] > 0.f ? 1.0f / ls[rs] : 0.f;
                        if (prm.o_f32)
                            *reinterpret_cast<float2*>(static_cast<float*>(prm.o) + hrow * D + n * 8 + qcol) =
                                make_float2(acc[2 * rs] * inv, acc[2 * rs + 1] * inv);
                        else
                            *reinterpret_cast<__half2*>(static_cast<__half*>(prm.o) + hrow * D + n * 8 + qcol) =
                                __floats2half2_rn(acc[2 * rs] * inv, acc[2 * rs + 1] * inv);
                    }
                }
            };
            auto emit_ml = [&](const float (&ms)[2], const float (&ls)[2]) {
                if ((PEER || prm.o_partial) && warp == 0 && (lane & 3) == 0) {
#pragma unroll
                    for (int rs = 0; rs < ROWSETS; ++rs) {
                        const uint32_t row = qrow + 8 * rs;
                        if (row >= prm.G) continue;
                        const size_t hrow = static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G + row;
                        if constexpr (PEER) {
                            peer_store_ml(hrow, ms[rs] * 0.6931471805599453f, ls[rs]);   // natural-log units, as in the caller-visible partial
                        } else {
                            prm.ml_partial[hrow * 2] = ms[rs] * 0.6931471805599453f;   // natural-log units for the caller
                            prm.ml_partial[hrow * 2 + 1] = ls[rs];
                        }
                    }
                }
            };
            using FragT = typename std::conditional<G16, float4, float2>::type;
#pragma unroll
            for (int nn = 0; nn < (NT_O + W - 1) / W; ++nn) {
                const int n = nn * W + static_cast<int>(warp);  // this warp's output n-tiles
                if (NT_O % W != 0 && n >= NT_O) break;
                float acc[FR];
#pragma unroll
                for (int f = 0; f < FR; ++f) acc[f] = 0.f;
#pragma unroll
                for (int k = 0; k < W; ++k)
#pragma unroll
                    for (int f = 0; f < FR; ++f) acc[f] += xb[k * kXWarpFloats + (n * 32 + lane) * FR + f] * wk[k][f >> 1];
                if (n_parts > 1) {
                    // a (request, head) cut over CTAs: this CTA's part goes to the workspace, fragment order
                    FragT* wo = reinterpret_cast<FragT*>(prm.work_o) + (static_cast<size_t>(part_slot) * NT_O + n) * 32 + lane;
                    if constexpr (G16) *wo = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    else *wo = make_float2(acc[0], acc[1]);
                } else {
                    emit(n, acc, lstar);
                }
            }
            if (n_parts > 1) {
                if (warp == 0) {
                    FragT* wm = reinterpret_cast<FragT*>(prm.work_ml) + static_cast<size_t>(part_slot) * 32 + lane;
                    if constexpr (G16) *wm = make_float4(mstar[0], lstar[0], mstar[1], lstar[1]);
                    else *wm = make_float2(mstar[0], lstar[0]);
                }
                // Publish and count: the CTA meets (its stores then happen before whatever thread 0 does next),
                // thread 0 adds 1 to the (request, head)'s counter with release + acquire semantics at GPU
                // scope - cumulative, so the whole CTA's stores are visible to whoever sees the count, and the
                // other parts' stores to this CTA after the second barrier. Whoever brings the last part
                // combines all of them; nobody waits for another CTA. The last arrival also puts the counter
                // back to 0 for the next launch (which cannot touch it before this grid has ended: its
                // arrivals come after griddepcontrol.wait).
                asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
                if (threadIdx.x == 0) {
                    uint32_t* c = prm.seg_counters + d1.y;
                    uint32_t before;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(c) : "memory");
                    const bool last = before + 1 == n_parts;
                    if (last) *c = 0u;
                    last_part_flag = last ? 1u : 0u;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
                if (last_part_flag) {
                    const uint32_t first_slot = d1.x;
                    const FragT* pm = reinterpret_cast<const FragT*>(prm.work_ml) + static_cast<size_t>(first_slot) * 32 + lane;
                    // One pass over the parts in slot order (the result does not depend on who arrived last),
                    // running maximum as in the tile loop: the (m, l) and the o fragments of a part are loaded
                    // together, so the pass costs one trip to L2 per few parts rather than two.
                    constexpr int NN = (NT_O + W - 1) / W;   // output n-tiles of this warp
                    float ms[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f};
                    float cacc[NN][FR];
#pragma unroll
                    for (int nn = 0; nn < NN; ++nn)
#pragma unroll
                        for (int f = 0; f < FR; ++f) cacc[nn][f] = 0.f;
                    const FragT* po = reinterpret_cast<const FragT*>(prm.work_o) + (static_cast<size_t>(first_slot) * NT_O + warp) * 32 + lane;
                    // the loads of CHUNK parts are issued before the first is used (each is a trip to L2)
                    constexpr int kPartFloats = FR * (1 + NN);
                    constexpr int CHUNK = 48 / kPartFloats >= 8 ? 8 : (48 / kPartFloats >= 4 ? 4 : 2);
                    for (uint32_t k0 = 0; k0 < n_parts; k0 += CHUNK) {
                        FragT mv[CHUNK], ov[CHUNK][NN];
#pragma unroll
                        for (int i = 0; i < CHUNK; ++i) {
                            const uint32_t k = k0 + i;
                            const bool valid = k < n_parts;
                            mv[i] = FragT{};
                            if (valid) mv[i] = __ldcg(pm + k * 32);
                            else mv[i].x = -INFINITY;   // skipped below
                            if constexpr (G16) { if (!valid) reinterpret_cast<float*>(&mv[i])[2] = -INFINITY; }
#pragma unroll
                            for (int nn = 0; nn < NN; ++nn) {
                                const int n = nn * W + static_cast<int>(warp);
                                ov[i][nn] = FragT{};
                                if (valid && (NT_O % W == 0 || n < NT_O)) ov[i][nn] = __ldcg(po + (static_cast<size_t>(k) * NT_O + nn * W) * 32);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < CHUNK; ++i) {
#pragma unroll
                            for (int rs = 0; rs < ROWSETS; ++rs) {
                                const float mk = reinterpret_cast<const float*>(&mv[i])[2 * rs];
                                const float lk = reinterpret_cast<const float*>(&mv[i])[2 * rs + 1];
                                if (mk == -INFINITY) continue;   // a part without a valid token (or past the end) weighs nothing
                                const float m_new = fmaxf(ms[rs], mk);
                                const float alpha = ex2(ms[rs] - m_new), w = ex2(mk - m_new);   // ex2(-inf) = 0 for the first part
                                ms[rs] = m_new;
                                ls[rs] = ls[rs] * alpha + lk * w;
#pragma unroll
                                for (int nn = 0; nn < NN; ++nn) {
                                    const float* o2 = reinterpret_cast<const float*>(&ov[i][nn]) + 2 * rs;
                                    cacc[nn][2 * rs] = cacc[nn][2 * rs] * alpha + o2[0] * w;
                                    cacc[nn][2 * rs + 1] = cacc[nn][2 * rs + 1] * alpha + o2[1] * w;
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int nn = 0; nn < NN; ++nn) {
                        const int n = nn * W + static_cast<int>(warp);
                        if (NT_O % W != 0 && n >= NT_O) break;
                        emit(n, cacc[nn], ls);
                    }
                    emit_ml(ms, ls);
                }
            } else {
                emit_ml(mstar, lstar);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");  // the exchange area is free for the next (request, head)
            if constexpr (PEER) {
                // this CTA wrote the (request, head)'s final rows: alone, or as the last of the CTAs it was cut over
                if (n_parts == 1 || last_part_flag)
                    peer_finish(static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G);
            }
            if (pi == 0) stamp(4);
        } else if (n_parts > 1) {
            // un-normalised partial -> workspace, fragment order (coalesced). The merge kernel
            // that follows in the stream reads it; the kernel boundary orders the two.
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
            if (prm.seg_counters) {
                // Publish: the warp's stores, a warp barrier (orders them before lane 0's next
                // operation), then a release reduction on the segment's counter for this warp -
                // fire and forget, nothing waits for a return value.
                __syncwarp();
                if (lane == 0) {
                    uint32_t* c = prm.seg_counters + static_cast<size_t>(d1.y) * kDecodeWarps + warp;
                    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c) : "memory");
                }
            }
            if (pi == 0) stamp(4);
        } else {
            write_rows<D, G16>(prm, req, head, lane, o_acc, m_run, l_run);
        }
        if (pi + 1 == n_pieces) stamp(7);
    }

    if (UNIT && dead) {
        // this warp gave up on a copy: it still meets its CTA's two barriers per remaining piece
        for (; pi < n_pieces; ++pi) {
            const uint4 dd = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi) + 1);
            asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
            if ((dd.z & 0xffffu) > 1u) {  // a cut (request, head): the CTA still counts its arrival
                asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
                if (threadIdx.x == 0) {
                    uint32_t* c = prm.seg_counters + dd.y;
                    uint32_t before;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(c) : "memory");
                    if (before + 1 == (dd.z & 0xffffu)) *c = 0u;
                    last_part_flag = 0u;  // nothing is combined from a piece that gave up
                }
                asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
            }
            asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
        }
    }

    // ---- in-kernel merge of the split segments: segment s belongs to CTA s mod gridDim ----
    // Every CTA of this grid is resident (the grid is at most one CTA per SM and at most two
    // grids overlap), so the pieces a merger waits for are running or done. The wait is bounded.
    if (prm.seg_counters && !dead) {
        for (uint32_t seg = cta; seg < prm.n_segs; seg += gridDim.x) {
            const uint4 sdw = __ldg(reinterpret_cast<const uint4*>(prm.seg_desc) + seg);
            SegDesc sd;
            sd.req = sdw.x; sd.hb = sdw.y; sd.first_slot = sdw.z; sd.n_parts = sdw.w;
            if (sd.hb * kDecodeWarps + warp >= prm.KVH) continue;
            uint32_t* c = prm.seg_counters + static_cast<size_t>(seg) * kDecodeWarps + warp;
            uint32_t seen = 0;
            if (lane == 0) {
                for (uint32_t i = 0; i < (1u << 20); ++i) {
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c) : "memory");
                    if (v >= sd.n_parts) {
                        seen = 1;
                        break;
                    }
                }
                if (seen) *c = 0;  // ready for the next launch (which starts publishing only after this grid is done)
                else atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT);
            }
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (!seen) continue;
            merge_segment<D, G16, true>(prm, sd, warp, lane);
        }
        stamp(5);
    }
    if constexpr (PEER) {
        // the last CTA to finish advances the step counter (graph replays need no host argument)
        asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(pp->done, 1u) == gridDim.x - 1) {
                *pp->done = 0;
                __threadfence();
                *reinterpret_cast<volatile uint32_t*>(pp->seq) = peer_step + 1u;
            }
        }
    }
}

template <int D, bool G16, bool UNIT>
__global__ void __launch_bounds__((UNIT ? unit_warps(D) : kDecodeWarps) * 32, 1)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const DecodeParams prm) {
    decode_layer_body<D, G16, UNIT, false>(tmK, tmV, prm, nullptr);
}

// Partial attention over this rank's slice of the pages + exchange + combine, one launch (unit-mode plans).
template <int D, bool G16>
__global__ void __launch_bounds__(unit_warps(D) * 32, 1)
paged_decode_exchange_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                             const DecodeParams prm, const PeerParams pp) {
    decode_layer_body<D, G16, true, true>(tmK, tmV, prm, &pp);
}

// ------------------------------------------------------------------------------
// every layer of a pass in one launch
// ------------------------------------------------------------------------------
// The body of the whole-pass launch (instantiated with UNIT = PASS = true; the flags keep the places visible
// where it differs from the per-layer kernel above).
// ONE launch runs every layer of a decode pass. The plan is the one of a single layer (the layers share their
// page tables), with its CTAs in descending order of load ("ranks"). A CTA item is a (request, group of hpc
// adjacent KV heads): warp w holds head w % hpc of the group and part w / hpc of that head's tiles, so that the
// warps of a CTA fetch hpc adjacent 128-byte chunks of every token row at about the same time - whole rows
// when hpc = KVH - which the memory system serves ~13 % faster than one head's chunks alone (measured).
// The n_layers x gridDim (layer, rank) items, listed rank-major - i.e. heaviest first - are dealt to the
// CTAs in serpentine order, one per CTA and round: in round j CTA c takes item j * gridDim + c (even j) or
// j * gridDim + gridDim - 1 - c (odd j), item k being (rank k / n_layers, layer k % n_layers). Every CTA thus
// gets n_layers items whose loads add up to nearly the same, whatever the spread inside a layer, and the
// grid has no tail per layer. Nothing is exchanged between CTAs; a warp's TMA ring runs on across the item
// boundaries. The layers must be independent of one another (all inputs ready when the launch starts).
template <int D, bool G16, bool UNIT, bool PASS>
__device__ __forceinline__ void decode_body(const CUtensorMap* tmK, const CUtensorMap* tmV, const LayerArgs* layers,
                                            const DecodeParams& prm) {
    constexpr int TOK = kTileTokens;
    constexpr int NT_S = TOK / 8;          // score n-tiles per tile
    constexpr int KSTEPS = D / 16;         // k-steps of Q.K^T
    constexpr int NT_O = D / 8;            // output n-tiles
    constexpr int SUBS = D / 64;           // 64-half boxes per row
    constexpr uint32_t kTileBytes = TOK * D * 2;       // one of K or V
    constexpr uint32_t kStageBytes = 2 * kTileBytes;
    constexpr int ROWSETS = G16 ? 2 : 1;
    constexpr int W = UNIT ? unit_warps(D) : kDecodeWarps;  // warps of this CTA
    static_assert(!PASS || UNIT, "a whole-pass launch runs unit-mode plans");

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[W][8];
    __shared__ uint32_t last_part_flag;  // unit mode: this CTA brought the last piece of a (request, head) cut over CTAs

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = blockIdx.x;
    const uint32_t stages = prm.stages;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ring = smem_base + warp * stages * kStageBytes;

    // ---- the items of this CTA: one per round. Without PASS there is one round: the CTA's own plan slice.
    const uint32_t n_rounds = PASS ? prm.n_layers : 1u;
    auto round_item = [&](uint32_t j, uint32_t& rank, uint32_t& layer) {
        if constexpr (PASS) {
            const uint32_t V = gridDim.x;
            const uint32_t k = j * V + ((j & 1u) ? V - 1u - cta : cta);
            rank = k / prm.n_layers;
            layer = k - rank * prm.n_layers;
        } else {
            rank = cta;
            layer = 0;
        }
    };
    auto slice_of = [&](uint32_t rank) -> uint32_t { return UNIT ? rank * W + warp : rank; };  // unit mode: one plan slice per warp

    // ---- issue side: walks this warp's tile lists, item after item, ahead of the consume side ----
    // Every read of the plan it needs is taken one step ahead of its use - the next item's tile count and
    // first 32 tile words (one per lane) while the current item is being fetched, the next 32 words of a long
    // list while the current 32 are in use - so that no tile waits on a trip to global memory for its word.
    uint32_t iss_round = 0, iss_pos = 0, iss_n = 0, iss_layer = 0;
    const uint32_t* iss_tiles = prm.tile_pages;
    uint32_t win_base = 0, win = 0, win_nx = 0;
    uint32_t pf_n = 0, pf_win = 0, pf_layer = 0;      // the following item, prefetched
    const uint32_t* pf_tiles = prm.tile_pages;
    auto iss_prefetch = [&](uint32_t j) {
        uint32_t rank;
        round_item(j, rank, pf_layer);
        pf_n = 0;
        if (PASS && rank >= prm.plan_ctas) return;   // a rank without work in this plan
        const uint32_t slice = slice_of(rank);
        pf_tiles = prm.tile_pages + static_cast<size_t>(slice) * prm.max_tiles;
        // independent loads (one memory round trip). The planner pads the arrays so that the 32-word read
        // stays inside the plan image.
        pf_n = __ldg(prm.cta_counts + 2 * slice + 1);
        pf_win = __ldg(pf_tiles + lane);
    };
    auto iss_open = [&](uint32_t j) {   // item j was prefetched
        iss_round = j;
        iss_pos = 0;
        win_base = 0;
        iss_layer = pf_layer;
        iss_tiles = pf_tiles;
        iss_n = pf_n;
        win = pf_win;
        // unconditional (the plan image is padded for it): a test on the count would make this load wait for
        // the count's own trip to memory in the prologue
        win_nx = __ldg(iss_tiles + 32u + lane);
        if (j + 1u < n_rounds) iss_prefetch(j + 1u);
    };
    // the next tile word to fetch, if any is left (moves on to the next item's list when one is used up)
    auto iss_peek = [&](uint32_t& e) -> bool {
        while (iss_pos >= iss_n) {
            if (iss_round + 1u >= n_rounds) return false;
            iss_open(iss_round + 1u);
        }
        if (iss_pos - win_base >= 32u) {  // uniform across the warp; positions advance by one
            win_base += 32u;
            win = win_nx;
            if (win_base + 32u < iss_n) win_nx = (win_base + 32u + lane < iss_n) ? __ldg(iss_tiles + win_base + 32u + lane) : 0u;
        }
        e = __shfl_sync(0xffffffffu, win, iss_pos - win_base);
        return true;
    };

    // Consume side of the first deal: counts and the first 16 piece descriptors (half a descriptor per lane),
    // read together with the issue side's loads.
    uint32_t c_rank, c_layer;
    round_item(0, c_rank, c_layer);
    iss_prefetch(0);
    const bool first_has_work = !(PASS && c_rank >= prm.plan_ctas);
    uint32_t n_pieces = 0;
    uint4 desc_half = make_uint4(0u, 0u, 0u, 0u);
    const PieceDesc* my_pieces = prm.pieces;
    const uint32_t* my_tiles = prm.tile_pages;
    if (first_has_work) {
        const uint32_t slice = slice_of(c_rank);
        my_pieces = prm.pieces + static_cast<size_t>(slice) * prm.max_pieces;
        my_tiles = prm.tile_pages + static_cast<size_t>(slice) * prm.max_tiles;
        n_pieces = __ldg(prm.cta_counts + 2 * slice);
        desc_half = __ldg(reinterpret_cast<const uint4*>(my_pieces) + lane);
    }
    iss_open(0);   // after the loads above have been issued: all of the prologue's plan reads share one trip to memory
    auto stamp = [&](int i) {
        if (prm.trace && lane == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            prm.trace[(static_cast<size_t>(cta) * W + warp) * 8 + i] = t;
        }
    };
    stamp(0);

    if (lane == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(smem_u32(&bars[warp][s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // Ring position counters of this warp. They count only tiles of head blocks in
    // which this warp owns a KV head, in the (identical) order of issue and use.
    // (kept as wrapping stage indices and a parity bit: the ring depth is a run-time value, and a
    // division by it per tile costs tens of instructions)
    uint32_t iss_stage = 0, con_stage = 0, con_parity = 0;
    // Issues the TMA copies of the tile word `e` (of layer `layer` in a whole-pass launch) into the next ring stage.
    auto issue_word = [&](uint32_t e, uint32_t layer) {
        const uint32_t hfield = (e >> kTileHbShift) & kTileHbMask;   // head block, or the head itself in unit mode
        const uint32_t head = UNIT ? hfield : hfield * kDecodeWarps + warp;
        if (!UNIT && head >= prm.KVH) return;  // this warp has no KV head in that head block
        const uint32_t s = iss_stage;
        iss_stage = (iss_stage + 1 == stages) ? 0u : iss_stage + 1;
        if (lane == 0) {
            const uint32_t bar = smem_u32(&bars[warp][s]);
            const uint32_t dst = ring + s * kStageBytes;
            const int page = static_cast<int>(e & kTilePageMask);
            const int slot0 = static_cast<int>(((e >> kTileSubShift) & 7u) * TOK);
            const CUtensorMap* mk = PASS ? &layers[layer].map_k : tmK;
            const CUtensorMap* mv = PASS ? &layers[layer].map_v : tmV;
            const bool pair = PASS ? layers[layer].kv_pair != 0u : prm.kv_pair != 0u;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, kStageBytes);
            if (D == 64 && pair) {
                tma_load_5d(dst, mk, bar, 0, static_cast<int>(head), slot0, page, 0);
            } else {
#pragma unroll
                for (int sub = 0; sub < SUBS; ++sub) {
                    tma_load_4d(dst + sub * (TOK * 128), mk, bar, sub * 64, static_cast<int>(head), slot0, page);
                    tma_load_4d(dst + kTileBytes + sub * (TOK * 128), mv, bar, sub * 64, static_cast<int>(head), slot0, page);
                }
            }
        }
    };

    // Prefetches run ahead over piece (and item) boundaries; they need nothing but the tile lists.
    // In a decode step, tiles that hold a row written in this step ("fresh" tiles: the
    // ones containing the new token) are not fetched before griddepcontrol.wait;
    // everything older may be.
    uint32_t in_flight = 0;   // tiles issued into the ring at start-up (at most the ring depth)
    if (prm.pdl) {
        if (prm.step && prm.early_fetch) {
            uint32_t e;
            while (in_flight < stages && iss_peek(e)) {
                if (e & kTileFreshBit) break;
                issue_word(e, iss_layer);
                ++iss_pos;
                ++in_flight;
            }
        }
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    {
        uint32_t e;
        while (in_flight < stages && iss_peek(e)) {
            issue_word(e, iss_layer);
            ++iss_pos;
            ++in_flight;
        }
    }
    stamp(1);

    // Requests that attend to nothing: their O rows are zeros (mm:2254-2257).
    for (uint32_t i = cta; i < prm.n_zero * n_rounds; i += gridDim.x) {
        const uint32_t r = prm.zero_rows[i % prm.n_zero];
        void* o_ptr = PASS ? layers[i / prm.n_zero].o : prm.o;
        for (uint32_t e = threadIdx.x; e < prm.H * D; e += blockDim.x) {
            const size_t idx = static_cast<size_t>(r) * prm.H * D + e;
            if (!PASS && prm.o_partial) {
                prm.o_partial[idx] = 0.f;
                if (e % D == 0) {
                    prm.ml_partial[(idx / D) * 2] = -INFINITY;
                    prm.ml_partial[(idx / D) * 2 + 1] = 0.f;
                }
            } else if (prm.o_f32) static_cast<float*>(o_ptr)[idx] = 0.f;
            else static_cast<__half*>(o_ptr)[idx] = __float2half_rn(0.f);
        }
    }

    const uint32_t qrow = lane >> 2, qcol = (lane & 3) * 2;
    // Per-lane byte offsets of the ldmatrix rows inside a swizzled tile, computed once: a K fragment of
    // score tile n, k-pair kp sits at koff[kp] + n * 1024, a V fragment of token block kt, column pair np
    // at voff[np] + kt * 2048 (the token index only enters through lane & 7 and a multiple of 8 rows).
    // Kept in registers at head_dim 64 (6 values); at 128 the kernel has none to spare and recomputes them.
    constexpr bool kKeepOffsets = (D == 64);
    auto k_offset = [&](int kp) -> uint32_t {
        const uint32_t chunk = kp * 4 + (lane >> 3);
        return (chunk >> 3) * (TOK * 128) + (lane & 7) * 128 + (((chunk & 7) ^ (lane & 7)) << 4);
    };
    auto v_offset = [&](int np) -> uint32_t {
        const uint32_t chunk = np * 2 + (lane >> 4);
        return (chunk >> 3) * (TOK * 128) + ((lane & 7) + ((lane >> 3) & 1) * 8) * 128 + (((chunk & 7) ^ (lane & 7)) << 4);
    };
    uint32_t koff[kKeepOffsets ? KSTEPS / 2 : 1], voff[kKeepOffsets ? NT_O / 2 : 1];
    if constexpr (kKeepOffsets) {
#pragma unroll
        for (int kp = 0; kp < KSTEPS / 2; ++kp) koff[kp] = k_offset(kp);
#pragma unroll
        for (int np = 0; np < NT_O / 2; ++np) voff[np] = v_offset(np);
    }
    // Unit mode: the warps that hold parts of this warp's head - all of them, or every hpc-th (a bit per warp) -
    // this warp's place among them and their number
    const uint32_t wgroup = UNIT ? W / prm.hpc : 1u, wpart = UNIT ? warp / prm.hpc : 0u;
    uint32_t same_head_mask = 0;
#pragma unroll
    for (int k = 0; k < W; ++k)
        if (prm.hpc == 1u || static_cast<uint32_t>(k) % prm.hpc == warp % prm.hpc) same_head_mask |= 1u << k;
    // A warp whose bounded wait ran out is `dead`: it records the error, fetches and computes nothing more, but
    // keeps walking its pieces so that it still meets its CTA's barriers (its parts weigh nothing).
    bool dead = false;
    // Look-ahead of the consume side. A piece starts with two dependent trips to memory (its descriptor, then
    // the Q rows the descriptor names) before its first MMA; both are taken one piece ahead - across item
    // boundaries too - wherever registers allow (head_dim 64).
    constexpr bool kLookAhead = PASS && D == 64;   // (in a launch per layer a CTA mostly has one piece: nothing to look ahead to)
    // Whole-pass launch: the next piece's Q block is copied into shared memory (cp.async, 16 bytes per thread,
    // the CTA's threads together) while the current piece runs, and a piece's O block is put together in shared
    // memory and written out by all threads in 16-byte pieces. Two Q buffers (current / next), one O buffer,
    // behind the exchange area of the in-CTA merge.
    constexpr bool kStageQ = kLookAhead;
    constexpr bool kStageO = PASS;
    constexpr uint32_t kXchgBytes = UNIT ? static_cast<uint32_t>(W) * (NT_O + 1) * 32 * (G16 ? 4 : 2) * 4 : 0;
    uint8_t* const io_base = smem_raw + (smem_base - smem_u32(smem_raw)) + static_cast<size_t>(W) * stages * kStageBytes + kXchgBytes;
    uint8_t* const o_stage = io_base + 2u * prm.q_block_bytes;
    uint32_t q_sel = 0;            // the Q buffer the next prefetch goes to
    uint32_t nx_rank = 0, nx_layer = 0, nx_pieces = 0;
    uint4 nx_desc_half = make_uint4(0u, 0u, 0u, 0u);
    bool pre_valid = false;          // pre_d0 / pre_d1 / pre_qa hold the piece about to start
    uint4 pre_d0 = make_uint4(0u, 0u, 0u, 0u), pre_d1 = pre_d0;
    uint32_t pre_qa[kLookAhead ? KSTEPS : 1][4];
    auto desc_from = [&](const uint4& halves, uint32_t i, uint4& a, uint4& b) {   // piece i < 16 of a prefetched list
        a.x = __shfl_sync(0xffffffffu, halves.x, 2 * i);
        a.y = __shfl_sync(0xffffffffu, halves.y, 2 * i);
        a.z = __shfl_sync(0xffffffffu, halves.z, 2 * i);
        a.w = __shfl_sync(0xffffffffu, halves.w, 2 * i);
        b.x = __shfl_sync(0xffffffffu, halves.x, 2 * i + 1);
        b.y = __shfl_sync(0xffffffffu, halves.y, 2 * i + 1);
        b.z = __shfl_sync(0xffffffffu, halves.z, 2 * i + 1);
        b.w = __shfl_sync(0xffffffffu, halves.w, 2 * i + 1);
    };
    // Q fragments (A operand) of one (request, KV head): rows = the query heads of the head's group
    auto load_q = [&](const void* q_base, uint32_t req, uint32_t head, uint32_t (&qa)[KSTEPS][4]) {
        const size_t q_row0 = (static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G) * D;
        const uint32_t qrow_ = lane >> 2, qcol_ = (lane & 3) * 2;
#pragma unroll
        for (int rs = 0; rs < 2; ++rs) {
            const uint32_t row = qrow_ + 8 * rs;
            const bool live = (rs < ROWSETS) && row < prm.G;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    uint32_t v = 0;
                    if (live) {
                        const size_t idx = q_row0 + static_cast<size_t>(row) * D + kk * 16 + hh * 8 + qcol_;
                        if (prm.q_f32) {
                            const float2 f = *reinterpret_cast<const float2*>(static_cast<const float*>(q_base) + idx);
                            v = pack_half2(f.x, f.y);
                        } else {
                            v = *reinterpret_cast<const uint32_t*>(static_cast<const __half*>(q_base) + idx);
                        }
                    }
                    qa[kk][rs + 2 * hh] = v;
                }
            }
        }
    };

  for (uint32_t round = 0; round < n_rounds; ++round) {
    // ---- per item: the slice's piece list and, in a whole-pass launch, the layer's buffers
    const void* q_ptr = prm.q;
    void* o_ptr = prm.o;
    const __half *k_new_ptr = prm.k_new, *v_new_ptr = prm.v_new;
    __half *k_pool_ptr = prm.k_pool, *v_pool_ptr = prm.v_pool;
    uint32_t k_off = prm.k_off, v_off = prm.v_off;
    if constexpr (PASS) {
        if (round > 0) {   // read while the round before was running
            c_rank = nx_rank;
            c_layer = nx_layer;
            n_pieces = nx_pieces;
            desc_half = nx_desc_half;
            if (c_rank < prm.plan_ctas) {
                const uint32_t slice = slice_of(c_rank);
                my_pieces = prm.pieces + static_cast<size_t>(slice) * prm.max_pieces;
                my_tiles = prm.tile_pages + static_cast<size_t>(slice) * prm.max_tiles;
            }
        }
        // the next round's piece count and first 16 descriptors: issued now, used a whole item later
        nx_pieces = 0;
        if (round + 1 < n_rounds) {
            round_item(round + 1, nx_rank, nx_layer);
            if (nx_rank < prm.plan_ctas) {
                const uint32_t slice = slice_of(nx_rank);
                nx_pieces = __ldg(prm.cta_counts + 2 * slice);
                nx_desc_half = __ldg(reinterpret_cast<const uint4*>(prm.pieces + static_cast<size_t>(slice) * prm.max_pieces) + lane);
            }
        }
        if (c_rank >= prm.plan_ctas) {   // the same for every warp of the CTA
            pre_valid = false;
            continue;
        }
        const LayerArgs& la = layers[c_layer];
        q_ptr = la.q; o_ptr = la.o;
        k_new_ptr = la.k_new; v_new_ptr = la.v_new;
        k_pool_ptr = la.k_pool; v_pool_ptr = la.v_pool;
        k_off = la.k_off; v_off = la.v_off;
    }
    uint32_t j = 0;  // tile counter within the slice (consume side)

    uint32_t pi = 0;
    for (; pi < n_pieces; ++pi) {
        uint4 d0, d1;
        const bool was_pre = kLookAhead && pre_valid;
        if (was_pre) {
            d0 = pre_d0;
            d1 = pre_d1;
        } else if (pi < 16u) {  // prefetched with the counts: lane 2i holds the first half of piece i
            desc_from(desc_half, pi, d0, d1);
        } else {
            d0 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi));
            d1 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi) + 1);
        }
        const uint32_t req = d0.x, piece_tiles = dead ? 0u : d0.z, part_slot = d0.w;
        const uint32_t n_parts = d1.z & 0xffffu, hb = d1.z >> 16;
        const uint32_t last_valid = d1.w & 0xffffu;
        const bool fresh_piece = prm.step && ((d1.w >> 16) & 1u);  // its last tile holds the new token
        const uint32_t head = UNIT ? hb : hb * kDecodeWarps + warp;
        if (head >= prm.KVH) {  // keep the tile counter and the prefetch stream in step
            for (uint32_t t = 0; t < piece_tiles; ++t, ++j) {
                uint32_t e;
                if (iss_peek(e)) {
                    issue_word(e, iss_layer);
                    ++iss_pos;
                }
            }
            continue;
        }

        // ---- Q fragments of this piece, and the look-ahead for the next one
        uint32_t qa[KSTEPS][4];
        if constexpr (kLookAhead) {
            if (was_pre && kStageQ) {
                // staged by the whole CTA during the piece before (complete and visible since that piece's
                // merge barrier): this warp's head is G rows inside the block
                const uint8_t* blk = io_base + (q_sel ^ 1u) * prm.q_block_bytes;
                const size_t esz = prm.q_f32 ? 4 : 2;
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
                                const size_t idx = (static_cast<size_t>(warp % prm.hpc) * prm.G + row) * D + kk * 16 + hh * 8 + qcol;
                                if (prm.q_f32) {
                                    const float2 f = *reinterpret_cast<const float2*>(blk + idx * esz);
                                    v = pack_half2(f.x, f.y);
                                } else {
                                    v = *reinterpret_cast<const uint32_t*>(blk + idx * esz);
                                }
                            }
                            qa[kk][rs + 2 * hh] = v;
                        }
                    }
                }
            } else if (was_pre) {
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk)
#pragma unroll
                    for (int i = 0; i < 4; ++i) qa[kk][i] = pre_qa[kk][i];
            } else {
                load_q(q_ptr, req, head, qa);
            }
            pre_valid = false;
            const void* nq_ptr = q_ptr;
            if (pi + 1 < n_pieces) {
                if (pi + 1 < 16u) {
                    desc_from(desc_half, pi + 1, pre_d0, pre_d1);
                } else {
                    pre_d0 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi + 1));
                    pre_d1 = __ldg(reinterpret_cast<const uint4*>(my_pieces + pi + 1) + 1);
                }
                pre_valid = true;
            } else if (PASS && nx_pieces > 0) {   // the first piece of the next item
                desc_from(nx_desc_half, 0, pre_d0, pre_d1);
                nq_ptr = layers[nx_layer].q;
                pre_valid = true;
            }
            if (pre_valid) {
                if constexpr (kStageQ) {
                    // the block of the next piece's head group: its hpc * G query heads are adjacent rows
                    const uint32_t nhead = pre_d1.z >> 16;
                    const size_t first_row = static_cast<size_t>(pre_d0.x) * prm.H + static_cast<size_t>(nhead - warp % prm.hpc) * prm.G;
                    const char* src = static_cast<const char*>(nq_ptr) + first_row * D * (prm.q_f32 ? 4 : 2);
                    const uint32_t dst = smem_u32(io_base + q_sel * prm.q_block_bytes);
                    for (uint32_t off = threadIdx.x * 16u; off < prm.q_block_bytes; off += blockDim.x * 16u)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + off), "l"(src + off) : "memory");
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    q_sel ^= 1u;
                } else {
                    load_q(nq_ptr, pre_d0.x, pre_d1.z >> 16, pre_qa);
                }
            }
        } else {
            load_q(q_ptr, req, head, qa);
        }
        // ---- decode step: this step's new K/V row of (request, head), one 16-byte chunk per
        // lane (lanes [0, D/8) hold K, lanes [16, 16 + D/8) hold V). It is written to the pool
        // here and patched over the fresh tile's copy in shared memory below.
        uint4 new_row = make_uint4(0u, 0u, 0u, 0u);
        constexpr uint32_t kRowChunks = D / 8;
        const bool row_lane = (lane & 15u) < kRowChunks;
        if (fresh_piece && row_lane) {
            const __half* src = (lane < 16u ? k_new_ptr : v_new_ptr) +
                                (static_cast<size_t>(req) * prm.KVH + head) * D + (lane & 15u) * 8;
            new_row = *reinterpret_cast<const uint4*>(src);
        }

        float o_acc[NT_O][4];
#pragma unroll
        for (int n = 0; n < NT_O; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        for (uint32_t t = 0; t < piece_tiles; ++t, ++j) {
            const uint32_t s = con_stage;
            const uint32_t bar = smem_u32(&bars[warp][s]);
            const uint32_t parity = con_parity;
            if (++con_stage == stages) {
                con_stage = 0;
                con_parity ^= 1u;
            }
            if (!mbar_wait_bounded(bar, parity)) {
                if (lane == 0) atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT);
                dead = true;
                break;
            }
            if (!PASS && j == 0) stamp(2);
            // the next tile word to fetch, taken now so that its shuffle (and every 32nd time the load of
            // the next window, or the opening of the next item's list) is long done when lane 0 needs it at
            // the end of the tile
            uint32_t e_next = 0u;
            const bool have_next = iss_peek(e_next);
            const uint32_t next_layer = iss_layer;
            const uint32_t sK = ring + s * kStageBytes + k_off, sV = ring + s * kStageBytes + v_off;
            const bool last_tile = t + 1 == piece_tiles;
            const uint32_t nv = last_tile ? last_valid : TOK;

            if (fresh_piece && last_tile) {
                // The new token is the last valid row of this tile; its pool address follows
                // from the tile word (page, sub-tile).
                const uint32_t rowi = nv - 1;
                const uint32_t e = __ldg(my_tiles + j);
                if (row_lane) {
                    const uint32_t chunk = lane & 15u;
                    const uint32_t addr = (lane < 16u ? sK : sV) + (chunk >> 3) * (TOK * 128) + rowi * 128 +
                                          (((chunk & 7) ^ (rowi & 7)) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(new_row.x), "r"(new_row.y),
                                 "r"(new_row.z), "r"(new_row.w) : "memory");
                    const size_t prow = (static_cast<size_t>(e & kTilePageMask) * prm.P +
                                         ((e >> kTileSubShift) & 7u) * TOK + rowi) * prm.KVH + head;
                    __half* dstp = (lane < 16u ? k_pool_ptr : v_pool_ptr) + prow * D + chunk * 8;
                    *reinterpret_cast<uint4*>(dstp) = new_row;
                }
                __syncwarp();
            }

            // ---- S = Q.K^T (fp32)
            // The shared-memory loads of a group of score tiles are all issued before the first MMA that
            // needs one (the asm statements keep their order, so load -> mma -> load -> mma would pay
            // the ldmatrix latency once per pair: ~1200 clocks per tile, measured), and the MMAs run
            // over independent accumulators in turn.
            float sc[NT_S][4];
            constexpr int kScoreGroup = (D == 64) ? NT_S : NT_S / 2;  // 32 fragment registers per group
#pragma unroll
            for (int n0 = 0; n0 < NT_S; n0 += kScoreGroup) {
                uint32_t kb[kScoreGroup][KSTEPS / 2][4];
#pragma unroll
                for (int kp = 0; kp < KSTEPS / 2; ++kp) {
                    const uint32_t addr = sK + (kKeepOffsets ? koff[kKeepOffsets ? kp : 0] : k_offset(kp)) + n0 * 1024;
                    static_assert(kScoreGroup <= 4, "unrolled by hand below");
                    ldsm_x4_off<0>(addr, kb[0][kp]);
                    if constexpr (kScoreGroup > 1) ldsm_x4_off<1024>(addr, kb[1][kp]);
                    if constexpr (kScoreGroup > 2) ldsm_x4_off<2048>(addr, kb[2][kp]);
                    if constexpr (kScoreGroup > 3) ldsm_x4_off<3072>(addr, kb[3][kp]);
                }
#pragma unroll
                for (int ni = 0; ni < kScoreGroup; ++ni) sc[n0 + ni][0] = sc[n0 + ni][1] = sc[n0 + ni][2] = sc[n0 + ni][3] = 0.f;
#pragma unroll
                for (int kp = 0; kp < KSTEPS / 2; ++kp) {
#pragma unroll
                    for (int ni = 0; ni < kScoreGroup; ++ni) mma_16816(sc[n0 + ni], qa[2 * kp], kb[ni][kp][0], kb[ni][kp][1]);
#pragma unroll
                    for (int ni = 0; ni < kScoreGroup; ++ni) mma_16816(sc[n0 + ni], qa[2 * kp + 1], kb[ni][kp][2], kb[ni][kp][3]);
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
                if (nv < TOK) {  // only a request's last tile is partly valid (warp-uniform)
#pragma unroll
                    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const uint32_t tok = n * 8 + qcol + e;
                            const float v = tok < nv ? sc[n][2 * rs + e] * prm.scale_log2 : -INFINITY;
                            sc[n][2 * rs + e] = v;
                            tmax = fmaxf(tmax, v);
                        }
                    }
                } else {
#pragma unroll
                    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float v = sc[n][2 * rs + e] * prm.scale_log2;
                            sc[n][2 * rs + e] = v;
                            tmax = fmaxf(tmax, v);
                        }
                    }
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run[rs], tmax);  // finite: every tile has >= 1 valid token
                float psum = 0.f;
#pragma unroll
                for (int n = 0; n < NT_S; ++n) {
                    const float p0 = ex2(sc[n][2 * rs] - m_new), p1 = ex2(sc[n][2 * rs + 1] - m_new);
                    psum += p0 + p1;
                    pa[n >> 1][rs + 2 * (n & 1)] = pack_half2(p0, p1);
                }
                // The accumulators are rescaled only when some row's maximum moved, which after the
                // first tiles of a request is rare (warp-uniform test).
                if (__any_sync(0xffffffffu, m_new > m_run[rs])) {
                    const float alpha = ex2(m_run[rs] - m_new);  // ex2(-inf) = 0 on the first tile
                    l_run[rs] *= alpha;
                    m_run[rs] = m_new;
#pragma unroll
                    for (int n = 0; n < NT_O; ++n) {
                        o_acc[n][2 * rs] *= alpha;
                        o_acc[n][2 * rs + 1] *= alpha;
                    }
                }
                l_run[rs] += psum;
            }
            if (!G16) {
#pragma unroll
                for (int kt = 0; kt < TOK / 16; ++kt) pa[kt][1] = pa[kt][3] = 0u;
            }

            // ---- O += P.V
            // same batching: the V fragments of 64 output columns first, then their MMAs
            constexpr int kOutGroup = 4;  // ldmatrix per batch = 16 fragment registers
#pragma unroll
            for (int kt = 0; kt < TOK / 16; ++kt) {
#pragma unroll
                for (int np0 = 0; np0 < NT_O / 2; np0 += kOutGroup) {
                    uint32_t vb[kOutGroup][4];
#pragma unroll
                    for (int i = 0; i < kOutGroup; ++i)
                        ldsm_x4_trans(sV + (kKeepOffsets ? voff[kKeepOffsets ? np0 + i : 0] : v_offset(np0 + i)) + kt * 2048, vb[i]);
#pragma unroll
                    for (int i = 0; i < kOutGroup; ++i) {
                        mma_16816(o_acc[2 * (np0 + i)], pa[kt], vb[i][0], vb[i][1]);
                        mma_16816(o_acc[2 * (np0 + i) + 1], pa[kt], vb[i][2], vb[i][3]);
                    }
                }
            }
            __syncwarp();
            if (have_next) {
                issue_word(e_next, next_layer);
                ++iss_pos;
            }
        }
        if (dead) {   // this piece's part (and every later one of this warp) weighs nothing
#pragma unroll
            for (int n = 0; n < NT_O; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
            m_run[0] = m_run[1] = -INFINITY;
            l_run[0] = l_run[1] = 0.f;
        }
        if (!PASS && pi == 0) stamp(3);

        // ---- end of piece: row sums over the quad
#pragma unroll
        for (int rs = 0; rs < ROWSETS; ++rs) {
            l_run[rs] += __shfl_xor_sync(0xffffffffu, l_run[rs], 1);
            l_run[rs] += __shfl_xor_sync(0xffffffffu, l_run[rs], 2);
        }

        if constexpr (kStageQ) asm volatile("cp.async.wait_group 0;" ::: "memory");   // the next piece's Q block (made visible by the barrier below)
        if (UNIT) {
            // The W warps hold the W parts of this (request, head): exchange the un-normalised
            // partials through shared memory, then every warp merges and writes its share of the
            // output columns.
            constexpr int FR = G16 ? 4 : 2;
            constexpr uint32_t kXWarpFloats = (NT_O + 1) * 32 * FR;
            float* xb = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) +
                        (static_cast<size_t>(W) * stages * kStageBytes) / 4;
            float* mine = xb + warp * kXWarpFloats;
#pragma unroll
            for (int n = 0; n < NT_O; ++n)
#pragma unroll
                for (int f = 0; f < FR; ++f) mine[(n * 32 + lane) * FR + f] = o_acc[n][f];
#pragma unroll
            for (int rs = 0; rs < ROWSETS; ++rs) {
                mine[(NT_O * 32 + lane) * FR + 2 * rs] = m_run[rs];
                mine[(NT_O * 32 + lane) * FR + 2 * rs + 1] = l_run[rs];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
            float wk[W][2], lstar[2], mstar[2];
#pragma unroll
            for (int rs = 0; rs < ROWSETS; ++rs) {
                float mk[W];
                mstar[rs] = -INFINITY;
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    const bool same_head = (same_head_mask >> k) & 1u;
                    mk[k] = same_head ? xb[k * kXWarpFloats + (NT_O * 32 + lane) * FR + 2 * rs] : -INFINITY;
                    mstar[rs] = fmaxf(mstar[rs], mk[k]);
                }
                lstar[rs] = 0.f;
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    wk[k][rs] = (mk[k] == -INFINITY) ? 0.f : ex2(mk[k] - mstar[rs]);  // an empty quarter weighs nothing
                    lstar[rs] += xb[k * kXWarpFloats + (NT_O * 32 + lane) * FR + 2 * rs + 1] * wk[k][rs];
                }
            }
            // Writes rows of O (or of the caller's partial output) for output n-tile n.
            auto emit = [&](int n, const float (&acc)[FR], const float (&ls)[2]) {
#pragma unroll
                for (int rs = 0; rs < ROWSETS; ++rs) {
                    const uint32_t row = qrow + 8 * rs;
                    if (row >= prm.G) continue;
                    const size_t hrow = static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G + row;
                    if (prm.o_partial) {
                        *reinterpret_cast<float2*>(prm.o_partial + hrow * D + n * 8 + qcol) = make_float2(acc[2 * rs], acc[2 * rs + 1]);
                    } else if (kStageO) {
                        // into the O block in shared memory: row (head inside the group) * G + row
                        const float inv = ls[rs] > 0.f ? 1.0f / ls[rs] : 0.f;
                        const size_t idx = (static_cast<size_t>(warp % prm.hpc) * prm.G + row) * D + n * 8 + qcol;
                        if (prm.o_f32)
                            *reinterpret_cast<float2*>(o_stage + idx * 4) = make_float2(acc[2 * rs] * inv, acc[2 * rs + 1] * inv);
                        else
                            *reinterpret_cast<__half2*>(o_stage + idx * 2) = __floats2half2_rn(acc[2 * rs] * inv, acc[2 * rs + 1] * inv);
                    } else {
                        const float inv = ls[rs] > 0.f ? 1.0f / ls[rs] : 0.f;
                        if (prm.o_f32)
                            *reinterpret_cast<float2*>(static_cast<float*>(o_ptr) + hrow * D + n * 8 + qcol) =
                                make_float2(acc[2 * rs] * inv, acc[2 * rs + 1] * inv);
                        else
                            *reinterpret_cast<__half2*>(static_cast<__half*>(o_ptr) + hrow * D + n * 8 + qcol) =
                                __floats2half2_rn(acc[2 * rs] * inv, acc[2 * rs + 1] * inv);
                    }
                }
            };
            auto emit_ml = [&](const float (&ms)[2], const float (&ls)[2]) {
                if (prm.o_partial && wpart == 0 && (lane & 3) == 0) {
#pragma unroll
                    for (int rs = 0; rs < ROWSETS; ++rs) {
                        const uint32_t row = qrow + 8 * rs;
                        if (row >= prm.G) continue;
                        const size_t hrow = static_cast<size_t>(req) * prm.H + static_cast<size_t>(head) * prm.G + row;
                        prm.ml_partial[hrow * 2] = ms[rs] * 0.6931471805599453f;   // natural-log units for the caller
                        prm.ml_partial[hrow * 2 + 1] = ls[rs];
                    }
                }
            };
            using FragT = typename std::conditional<G16, float4, float2>::type;
#pragma unroll 1
            for (int n = static_cast<int>(wpart); n < NT_O; n += static_cast<int>(wgroup)) {   // this warp's output n-tiles
                float acc[FR];
#pragma unroll
                for (int f = 0; f < FR; ++f) acc[f] = 0.f;
#pragma unroll
                for (int k = 0; k < W; ++k)
#pragma unroll
                    for (int f = 0; f < FR; ++f) acc[f] += xb[k * kXWarpFloats + (n * 32 + lane) * FR + f] * wk[k][f >> 1];
                if (n_parts > 1) {
                    // a (request, head) cut over CTAs: this CTA's part goes to the workspace, fragment order
                    FragT* wo = reinterpret_cast<FragT*>(prm.work_o) + (static_cast<size_t>(part_slot) * NT_O + n) * 32 + lane;
                    if constexpr (G16) *wo = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    else *wo = make_float2(acc[0], acc[1]);
                } else {
                    emit(n, acc, lstar);
                }
            }
            if (n_parts > 1) {
                if (warp == 0) {
                    FragT* wm = reinterpret_cast<FragT*>(prm.work_ml) + static_cast<size_t>(part_slot) * 32 + lane;
                    if constexpr (G16) *wm = make_float4(mstar[0], lstar[0], mstar[1], lstar[1]);
                    else *wm = make_float2(mstar[0], lstar[0]);
                }
                // Publish and count: the CTA meets (its stores then happen before whatever thread 0 does next),
                // thread 0 adds 1 to the (request, head)'s counter with release + acquire semantics at GPU
                // scope - cumulative, so the whole CTA's stores are visible to whoever sees the count, and the
                // other parts' stores to this CTA after the second barrier. Whoever brings the last part
                // combines all of them; nobody waits for another CTA. The last arrival also puts the counter
                // back to 0 for the next launch (which cannot touch it before this grid has ended: its
                // arrivals come after griddepcontrol.wait).
                asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
                if (threadIdx.x == 0) {
                    uint32_t* c = prm.seg_counters + d1.y;
                    uint32_t before;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(c) : "memory");
                    const bool last = before + 1 == n_parts;
                    if (last) *c = 0u;
                    last_part_flag = last ? 1u : 0u;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
                if (last_part_flag) {
                    const uint32_t first_slot = d1.x;
                    const FragT* pm = reinterpret_cast<const FragT*>(prm.work_ml) + static_cast<size_t>(first_slot) * 32 + lane;
                    // One pass over the parts in slot order (the result does not depend on who arrived last),
                    // running maximum as in the tile loop: the (m, l) and the o fragments of a part are loaded
                    // together, so the pass costs one trip to L2 per few parts rather than two.
                    constexpr int NN = (NT_O + W - 1) / W;   // output n-tiles of this warp
                    float ms[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f};
                    float cacc[NN][FR];
#pragma unroll
                    for (int nn = 0; nn < NN; ++nn)
#pragma unroll
                        for (int f = 0; f < FR; ++f) cacc[nn][f] = 0.f;
                    const FragT* po = reinterpret_cast<const FragT*>(prm.work_o) + (static_cast<size_t>(first_slot) * NT_O + warp) * 32 + lane;
                    // the loads of CHUNK parts are issued before the first is used (each is a trip to L2)
                    constexpr int kPartFloats = FR * (1 + NN);
                    constexpr int CHUNK = 48 / kPartFloats >= 8 ? 8 : (48 / kPartFloats >= 4 ? 4 : 2);
                    for (uint32_t k0 = 0; k0 < n_parts; k0 += CHUNK) {
                        FragT mv[CHUNK], ov[CHUNK][NN];
#pragma unroll
                        for (int i = 0; i < CHUNK; ++i) {
                            const uint32_t k = k0 + i;
                            const bool valid = k < n_parts;
                            mv[i] = FragT{};
                            if (valid) mv[i] = __ldcg(pm + k * 32);
                            else mv[i].x = -INFINITY;   // skipped below
                            if constexpr (G16) { if (!valid) reinterpret_cast<float*>(&mv[i])[2] = -INFINITY; }
#pragma unroll
                            for (int nn = 0; nn < NN; ++nn) {
                                const int n = nn * W + static_cast<int>(warp);
                                ov[i][nn] = FragT{};
                                if (valid && (NT_O % W == 0 || n < NT_O)) ov[i][nn] = __ldcg(po + (static_cast<size_t>(k) * NT_O + nn * W) * 32);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < CHUNK; ++i) {
#pragma unroll
                            for (int rs = 0; rs < ROWSETS; ++rs) {
                                const float mk = reinterpret_cast<const float*>(&mv[i])[2 * rs];
                                const float lk = reinterpret_cast<const float*>(&mv[i])[2 * rs + 1];
                                if (mk == -INFINITY) continue;   // a part without a valid token (or past the end) weighs nothing
                                const float m_new = fmaxf(ms[rs], mk);
                                const float alpha = ex2(ms[rs] - m_new), w = ex2(mk - m_new);   // ex2(-inf) = 0 for the first part
                                ms[rs] = m_new;
                                ls[rs] = ls[rs] * alpha + lk * w;
#pragma unroll
                                for (int nn = 0; nn < NN; ++nn) {
                                    const float* o2 = reinterpret_cast<const float*>(&ov[i][nn]) + 2 * rs;
                                    cacc[nn][2 * rs] = cacc[nn][2 * rs] * alpha + o2[0] * w;
                                    cacc[nn][2 * rs + 1] = cacc[nn][2 * rs + 1] * alpha + o2[1] * w;
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int nn = 0; nn < NN; ++nn) {
                        const int n = nn * W + static_cast<int>(warp);
                        if (NT_O % W != 0 && n >= NT_O) break;
                        emit(n, cacc[nn], ls);
                    }
                    emit_ml(ms, ls);
                }
            } else {
                emit_ml(mstar, lstar);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");  // the exchange area is free for the next (request, head)
            if constexpr (kStageO) {
                // the O block is complete: all threads write it out, 16 bytes each, rows of the head group adjacent
                const size_t first_row = static_cast<size_t>(req) * prm.H + static_cast<size_t>(head - warp % prm.hpc) * prm.G;
                char* dst = static_cast<char*>(o_ptr) + first_row * D * (prm.o_f32 ? 4 : 2);
                for (uint32_t off = threadIdx.x * 16u; off < prm.o_block_bytes; off += blockDim.x * 16u)
                    *reinterpret_cast<uint4*>(dst + off) = *reinterpret_cast<const uint4*>(o_stage + off);
            }
            if (pi == 0) stamp(4);
        } else if (n_parts > 1) {
            // un-normalised partial -> workspace, fragment order (coalesced). The merge kernel
            // that follows in the stream reads it; the kernel boundary orders the two.
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
            if (prm.seg_counters) {
                // Publish: the warp's stores, a warp barrier (orders them before lane 0's next
                // operation), then a release reduction on the segment's counter for this warp -
                // fire and forget, nothing waits for a return value.
                __syncwarp();
                if (lane == 0) {
                    uint32_t* c = prm.seg_counters + static_cast<size_t>(d1.y) * kDecodeWarps + warp;
                    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c) : "memory");
                }
            }
            if (pi == 0) stamp(4);
        } else {
            write_rows<D, G16>(prm, req, head, lane, o_acc, m_run, l_run);
        }
        if (pi + 1 == n_pieces) stamp(7);
    }

  }  // rounds

    // ---- in-kernel merge of the split segments: segment s belongs to CTA s mod gridDim ----
    // Every CTA of this grid is resident (the grid is at most one CTA per SM and at most two
    // grids overlap), so the pieces a merger waits for are running or done. The wait is bounded.
    if (prm.seg_counters && !dead) {
        for (uint32_t seg = cta; seg < prm.n_segs; seg += gridDim.x) {
            const uint4 sdw = __ldg(reinterpret_cast<const uint4*>(prm.seg_desc) + seg);
            SegDesc sd;
            sd.req = sdw.x; sd.hb = sdw.y; sd.first_slot = sdw.z; sd.n_parts = sdw.w;
            if (sd.hb * kDecodeWarps + warp >= prm.KVH) continue;
            uint32_t* c = prm.seg_counters + static_cast<size_t>(seg) * kDecodeWarps + warp;
            uint32_t seen = 0;
            if (lane == 0) {
                for (uint32_t i = 0; i < (1u << 20); ++i) {
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c) : "memory");
                    if (v >= sd.n_parts) {
                        seen = 1;
                        break;
                    }
                }
                if (seen) *c = 0;  // ready for the next launch (which starts publishing only after this grid is done)
                else atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT);
            }
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (!seen) continue;
            merge_segment<D, G16, true>(prm, sd, warp, lane);
        }
        stamp(5);
    }
}


// Every layer of a decode pass in one launch (see decode_body, PASS).
template <int D, bool G16>
__global__ void __launch_bounds__(unit_warps(D) * 32, 1)
paged_decode_pass_kernel(const __grid_constant__ PassArgs pass, const DecodeParams prm) {
    decode_body<D, G16, true, true>(nullptr, nullptr, pass.layer, prm);
}

// ------------------------------------------------------------------------------
// merging the pieces of a split (request, head block): one warp per KV head
// ------------------------------------------------------------------------------
// CG: read the partials with L1-bypassing loads. Needed when the merge runs inside the kernel
// that produced them (this SM's L1 may still hold lines of the same workspace from an earlier
// launch); a separate merge kernel starts with a clean L1.
template <typename T, bool CG>
__device__ __forceinline__ T ld_partial(const T* p) {
    if constexpr (CG) return __ldcg(p);
    else return *p;
}

template <int D, bool G16, bool CG>
__device__ __forceinline__ void merge_segment(const DecodeParams& prm, const SegDesc& sd, uint32_t warp, uint32_t lane) {
    constexpr int NT_O = D / 8;
    constexpr int ROWSETS = G16 ? 2 : 1;
    constexpr int FR = G16 ? 4 : 2;  // floats per lane per output n-tile
    constexpr int BATCH = (NT_O * FR) <= 16 ? 12 : ((NT_O * FR) <= 32 ? 6 : 3);
    const uint32_t head = sd.hb * kDecodeWarps + warp;
    float o_acc[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // One pass with a running maximum; the loads of a batch of partials are all issued
    // before any of them is used, so a batch costs a single L2 round trip.
    for (uint32_t k0 = 0; k0 < sd.n_parts; k0 += BATCH) {
        float mlb[BATCH][FR];
        float ob[BATCH][NT_O][FR];
#pragma unroll
        for (int bi = 0; bi < BATCH; ++bi) {
            const uint32_t k = (k0 + bi < sd.n_parts) ? k0 + bi : sd.n_parts - 1;
            const size_t u = static_cast<size_t>(sd.first_slot + k) * kDecodeWarps + warp;
            if (G16) {
                const float4 ml = ld_partial<float4, CG>(reinterpret_cast<const float4*>(prm.work_ml) + u * 32 + lane);
                mlb[bi][0] = ml.x; mlb[bi][1] = ml.y; mlb[bi][FR - 2] = ml.z; mlb[bi][FR - 1] = ml.w;
                const float4* wo = reinterpret_cast<const float4*>(prm.work_o) + u * NT_O * 32;
#pragma unroll
                for (int n = 0; n < NT_O; ++n) {
                    const float4 v = ld_partial<float4, CG>(wo + n * 32 + lane);
                    ob[bi][n][0] = v.x; ob[bi][n][1] = v.y; ob[bi][n][FR - 2] = v.z; ob[bi][n][FR - 1] = v.w;
                }
            } else {
                const float2 ml = ld_partial<float2, CG>(reinterpret_cast<const float2*>(prm.work_ml) + u * 32 + lane);
                mlb[bi][0] = ml.x; mlb[bi][1] = ml.y;
                const float2* wo = reinterpret_cast<const float2*>(prm.work_o) + u * NT_O * 32;
#pragma unroll
                for (int n = 0; n < NT_O; ++n) {
                    const float2 v = ld_partial<float2, CG>(wo + n * 32 + lane);
                    ob[bi][n][0] = v.x; ob[bi][n][1] = v.y;
                }
            }
        }
#pragma unroll
        for (int bi = 0; bi < BATCH; ++bi) {
            if (k0 + bi >= sd.n_parts) break;
#pragma unroll
            for (int rs = 0; rs < ROWSETS; ++rs) {
                const float mk = mlb[bi][2 * rs], lk = mlb[bi][2 * rs + 1];  // mk is finite
                const float m_new = fmaxf(m_run[rs], mk);
                const float a = ex2(m_run[rs] - m_new), w = ex2(mk - m_new);
                l_run[rs] = l_run[rs] * a + lk * w;
                m_run[rs] = m_new;
#pragma unroll
                for (int n = 0; n < NT_O; ++n) {
                    o_acc[n][2 * rs] = o_acc[n][2 * rs] * a + ob[bi][n][2 * rs] * w;
                    o_acc[n][2 * rs + 1] = o_acc[n][2 * rs + 1] * a + ob[bi][n][2 * rs + 1] * w;
                }
            }
        }
    }
    write_rows<D, G16>(prm, sd.req, head, lane, o_acc, m_run, l_run);
}

// The merge as a kernel of its own (one CTA per split segment), chained behind the attention
// kernel by programmatic dependent launch. Used when the launch has no arrival counters
// (caller-provided scratch).
template <int D, bool G16>
__global__ void __launch_bounds__(kDecodeWarps * 32)
paged_decode_merge_kernel(const DecodeParams prm) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The segment descriptor is plan data: read it while the attention kernel still runs.
    // Then let the next kernel in the stream start its own prologue, and wait until the
    // attention kernel that produced the partials has completed.
    const uint4 sdw = __ldg(reinterpret_cast<const uint4*>(prm.seg_desc) + blockIdx.x);
    SegDesc sd;
    sd.req = sdw.x; sd.hb = sdw.y; sd.first_slot = sdw.z; sd.n_parts = sdw.w;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (sd.hb * kDecodeWarps + warp >= prm.KVH) return;
    merge_segment<D, G16, false>(prm, sd, warp, lane);
}

// ------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------
static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

bool decode_tma_shape_supported(size_t H, size_t KVH, size_t D, size_t P, size_t capacity) {
    if (D != 64 && D != 128) return false;
    if (P % kTileTokens != 0 || P / kTileTokens > 8) return false;
    if (KVH == 0 || H / KVH > 16) return false;
    if ((KVH + kDecodeWarps - 1) / kDecodeWarps > kTileHbMask + 1) return false;
    if (capacity == 0 || capacity > kTilePageMask + size_t(1)) return false;
    return true;
}

bool decode_tma_pointers_supported(const AttnArgs& a) {
    if (!aligned(a.k_pages, 16) || !aligned(a.v_pages, 16)) return false;
    if (!aligned(a.q, a.q_dtype == MLC_F32 ? 8 : 4)) return false;
    if (a.o && !aligned(a.o, a.o_dtype == MLC_F32 ? 8 : 4)) return false;
    if (a.o_partial && (!aligned(a.o_partial, 8) || !a.ml_partial)) return false;
    if (a.k_new && (!aligned(a.k_new, 16) || !aligned(a.v_new, 16))) return false;
    return true;
}

// Deepest TMA ring that fits in the SM's shared memory.
uint32_t decode_tma_max_stages(size_t H, size_t KVH, size_t D) {
    (void)H; (void)KVH;
    const size_t stage = static_cast<size_t>(kDecodeWarps) * 2 * kTileTokens * D * 2;
    const size_t avail = 227 * 1024 - 2048;
    return static_cast<uint32_t>(std::min<size_t>(8, avail / stage));
}

// Shared memory of one CTA: the TMA rings, alignment slack and, in unit mode, the exchange
// area of the in-CTA merge (per warp (D/8 + 1) x 32 lanes x 2 or 4 floats).
size_t decode_tma_smem_bytes(size_t D, bool g16, uint32_t stages, bool unit) {
    const size_t warps = unit ? unit_warps(D) : kDecodeWarps;
    size_t smem = warps * stages * (2 * kTileTokens * D * 2) + 1024;
    if (unit) smem += warps * (D / 8 + 1) * 32 * (g16 ? 4 : 2) * 4;
    return smem;
}

template <int D, bool G16, bool UNIT>
static int launch_t(mlc_ctx* ctx, const DecodePlanView& plan, const DecodeParams& prm, const CUtensorMap& mk,
                    const CUtensorMap& mv) {
    const size_t smem = decode_tma_smem_bytes(D, G16, plan.stages, UNIT);
    size_t& configured = ctx->decode_smem_set[(UNIT ? 4 : 0) + (D == 128 ? 2 : 0) + (G16 ? 1 : 0)];
    if (smem > configured) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(paged_decode_tma_kernel<D, G16, UNIT>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured = smem;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.n_cta);
    cfg.blockDim = dim3((UNIT ? unit_warps(D) : kDecodeWarps) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = prm.pdl ? 1 : 0;
    MLCB_CUDA(ctx, cudaLaunchKernelEx(&cfg, paged_decode_tma_kernel<D, G16, UNIT>, mk, mv, prm));
    ++ctx->launches;
    if (plan.n_segs && !prm.seg_counters) {
        // the merge is always chained programmatically: before its wait it touches nothing
        cudaLaunchConfig_t mc{};
        mc.gridDim = dim3(plan.n_segs);
        mc.blockDim = dim3(kDecodeWarps * 32);
        mc.dynamicSmemBytes = 0;
        mc.stream = ctx->stream;
        mc.attrs = attr;
        mc.numAttrs = 1;
        MLCB_CUDA(ctx, cudaLaunchKernelEx(&mc, paged_decode_merge_kernel<D, G16>, prm));
        ++ctx->launches;
    }
    return MLC_OK;
}

template <int D, bool G16>
static int launch_exchange_t(mlc_ctx* ctx, const DecodePlanView& plan, const DecodeParams& prm, const CUtensorMap& mk,
                             const CUtensorMap& mv, const PeerParams& pp) {
    const size_t smem = decode_tma_smem_bytes(D, G16, plan.stages, true);
    size_t& configured = ctx->decode_smem_set[12 + (D == 128 ? 2 : 0) + (G16 ? 1 : 0)];
    if (smem > configured) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(paged_decode_exchange_kernel<D, G16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(smem)));
        configured = smem;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan.n_cta);      // at most one CTA per SM: every CTA of the launch is resident while it waits
    cfg.blockDim = dim3(unit_warps(D) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MLCB_CUDA(ctx, cudaLaunchKernelEx(&cfg, paged_decode_exchange_kernel<D, G16>, mk, mv, prm, pp));
    ++ctx->launches;
    return MLC_OK;
}

// True when one of the two decode launches enqueued before this one on the context writes into either pool.
static bool recently_written(const mlc_ctx* ctx, const void* k_pool, const void* v_pool) {
    for (const PoolWrites& w : ctx->recent_writes) {
        for (const void* p : w.few)
            if (p && (p == k_pool || p == v_pool)) return true;
        for (const void* p : w.many)
            if (p == k_pool || p == v_pool) return true;
    }
    return false;
}

void destroy_pass_args(mlc_ctx* ctx) {
    delete static_cast<PassArgs*>(ctx->pass_args);
    ctx->pass_args = nullptr;
}

template <int D, bool G16>
static int launch_pass_t(mlc_ctx* ctx, const DecodePlanView& plan, const DecodeParams& prm, const PassArgs& pass) {
    (void)plan;
    const size_t smem = decode_tma_smem_bytes(D, G16, prm.stages, true) + 2 * prm.q_block_bytes + prm.o_block_bytes;
    size_t& configured = ctx->decode_smem_set[8 + (D == 128 ? 2 : 0) + (G16 ? 1 : 0)];
    if (smem > configured) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(paged_decode_pass_kernel<D, G16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(smem)));
        configured = smem;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(ctx->sm_count));   // one CTA per SM, whatever the plan's CTA count
    cfg.blockDim = dim3(unit_warps(D) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MLCB_CUDA(ctx, cudaLaunchKernelEx(&cfg, paged_decode_pass_kernel<D, G16>, pass, prm));
    ++ctx->launches;
    return MLC_OK;
}

bool decode_pass_supported(const DecodePlanView& plan, size_t n_layers) {
    return plan.pass_ready && plan.has_tma && plan.unit_mode && plan.n_unit_cuts == 0 && plan.step_fusable && n_layers >= 2 &&
           n_layers <= static_cast<size_t>(kMaxPassLayers);
}

int launch_decode_pass_tma(mlc_ctx* ctx, const AttnArgs& shape, const DecodePlanView& plan, size_t n_layers,
                           const void* const* q, const void* const* k_new, const void* const* v_new,
                           void* const* k_pages, void* const* v_pages, void* const* o) {
    const uint32_t G = static_cast<uint32_t>(shape.H / shape.KVH);
    const bool g16 = G > 8;
    static const bool pair_allowed = [] {
        const char* v = std::getenv("MLC_B200_DECODE_KV_PAIR");
        return !(v && *v && std::atoi(v) == 0);
    }();
    // 20 KiB of kernel parameters, assembled in a buffer the context keeps (no allocation per call)
    if (!ctx->pass_args) ctx->pass_args = new PassArgs();
    PassArgs& pass = *static_cast<PassArgs*>(ctx->pass_args);
    const uint32_t tile_bytes = static_cast<uint32_t>(kTileTokens * shape.D * 2);
    for (size_t l = 0; l < n_layers; ++l) {
        AttnArgs a = shape;
        a.q = q[l]; a.o = o[l]; a.k_new = k_new[l]; a.v_new = v_new[l]; a.k_pages = k_pages[l]; a.v_pages = v_pages[l];
        if (!a.q || !a.o || !a.k_new || !a.v_new || !a.k_pages || !a.v_pages) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer in layer %zu", l);
        if (!decode_tma_pointers_supported(a)) return MLC_ERR_UNSUPPORTED;   // the caller falls back to per-layer launches
        LayerArgs& la = pass.layer[l];
        const bool kv_pair = pair_allowed && shape.D == 64 && pair_map_possible(a.k_pages, a.v_pages);
        int st;
        if (kv_pair) {
            if ((st = get_tensor_map(ctx, a.k_pages, a, &la.map_k, a.v_pages)) != MLC_OK) return st;
            la.map_v = la.map_k;
        } else {
            if ((st = get_tensor_map(ctx, a.k_pages, a, &la.map_k)) != MLC_OK) return st;
            if ((st = get_tensor_map(ctx, a.v_pages, a, &la.map_v)) != MLC_OK) return st;
        }
        const bool k_first = !kv_pair || reinterpret_cast<uintptr_t>(a.k_pages) < reinterpret_cast<uintptr_t>(a.v_pages);
        la.q = a.q; la.o = a.o;
        la.k_new = static_cast<const __half*>(a.k_new);
        la.v_new = static_cast<const __half*>(a.v_new);
        la.k_pool = static_cast<__half*>(const_cast<void*>(a.k_pages));
        la.v_pool = static_cast<__half*>(const_cast<void*>(a.v_pages));
        la.kv_pair = kv_pair ? 1u : 0u;
        la.k_off = k_first ? 0u : tile_bytes;
        la.v_off = k_first ? tile_bytes : 0u;
        la.pad = 0;
    }
    DecodeParams prm{};
    prm.cta_counts = plan.cta_counts;
    prm.pieces = plan.pieces;
    prm.tile_pages = plan.tile_pages;
    prm.zero_rows = plan.zero_rows;
    prm.seg_desc = plan.seg_desc;
    prm.err = ctx->d_err;
    prm.max_pieces = plan.max_pieces;
    prm.max_tiles = plan.max_tiles;
    prm.n_zero = plan.n_zero;
    prm.H = static_cast<uint32_t>(shape.H);
    prm.KVH = static_cast<uint32_t>(shape.KVH);
    prm.G = G;
    prm.P = static_cast<uint32_t>(shape.P);
    prm.scale_log2 = shape.scale * 1.4426950408889634f;
    prm.q_f32 = shape.q_dtype == MLC_F32;
    prm.o_f32 = shape.o_dtype == MLC_F32;
    prm.step = 1;
    prm.pdl = 1;
    // as in launch_attention_decode_tma: no fetch before the wait from a pool that one of the two decode
    // launches enqueued just before this one writes (here: any layer's pool)
    prm.early_fetch = 1;
    for (size_t l = 0; l < n_layers; ++l)
        if (recently_written(ctx, k_pages[l], v_pages[l])) prm.early_fetch = 0;
    ctx->recent_writes[0] = std::move(ctx->recent_writes[1]);
    ctx->recent_writes[1].few[0] = ctx->recent_writes[1].few[1] = nullptr;
    ctx->recent_writes[1].many.assign(k_pages, k_pages + n_layers);
    ctx->recent_writes[1].many.insert(ctx->recent_writes[1].many.end(), v_pages, v_pages + n_layers);
    prm.n_layers = static_cast<uint32_t>(n_layers);
    prm.plan_ctas = plan.n_cta;
    prm.hpc = plan.hpc ? plan.hpc : 1u;
    // Q / O blocks of a work item, staged through shared memory (Q only where the kernel looks a piece ahead)
    prm.q_block_bytes = shape.D == 64 ? static_cast<uint32_t>(prm.hpc * G * shape.D * (prm.q_f32 ? 4 : 2)) : 0u;
    prm.o_block_bytes = static_cast<uint32_t>(prm.hpc * G * shape.D * (prm.o_f32 ? 4 : 2));
    // Ring depth: what fits beside the staging buffers, at most MLC_B200_DECODE_PASS_STAGES (default 2 at
    // head_dim 64: with every SM streaming all the time a third stage measured 2 % slower, 22 layers x 32
    // requests; the plan's depth at 128)
    static const int pass_stages_env = [] {
        const char* v = std::getenv("MLC_B200_DECODE_PASS_STAGES");
        return v && *v ? std::atoi(v) : 0;
    }();
    prm.stages = pass_stages_env > 0 ? static_cast<uint32_t>(pass_stages_env) : (shape.D == 64 ? 2u : plan.stages);
    if (prm.stages > 8u) prm.stages = 8u;
    while (prm.stages > 1 && decode_tma_smem_bytes(shape.D, g16, prm.stages, true) + 2 * prm.q_block_bytes + prm.o_block_bytes > 227 * 1024 - 1024) --prm.stages;
    if (decode_tma_smem_bytes(shape.D, g16, prm.stages, true) + 2 * prm.q_block_bytes + prm.o_block_bytes > 227 * 1024 - 1024) return MLC_ERR_UNSUPPORTED;
    prm.trace = nullptr;
    ctx->trace_ctas = 0;
    if (shape.D == 64) return g16 ? launch_pass_t<64, true>(ctx, plan, prm, pass) : launch_pass_t<64, false>(ctx, plan, prm, pass);
    return g16 ? launch_pass_t<128, true>(ctx, plan, prm, pass) : launch_pass_t<128, false>(ctx, plan, prm, pass);
}

int launch_attention_decode_tma(mlc_ctx* ctx, const AttnArgs& a, const DecodePlanView& plan) {
    const uint32_t G = static_cast<uint32_t>(a.H / a.KVH);
    const bool g16 = G > 8;
    const bool step = a.k_new != nullptr;
    const size_t frag_floats = (g16 ? 4 : 2) * 32 * (a.D / 8);  // per (slot, warp)
    const size_t ml_floats = (g16 ? 4 : 2) * 32;
    const size_t units = static_cast<size_t>(plan.n_slots) * kDecodeWarps;
    const size_t o_bytes = ((units * frag_floats * 4 + 255) / 256) * 256;
    const size_t ml_bytes = ((units * ml_floats * 4 + 255) / 256) * 256;
    // Two copies of the workspace, used alternately: with programmatic dependent launch
    // the next attention kernel may publish partials while this one's merge still reads.
    int st = MLC_OK;
    CUtensorMap mk, mv;
    char* work = nullptr;
    uint32_t parity = 0;
    bool use_counters = false;
    uint32_t* ext_counters = nullptr;
    // MLC_B200_DECODE_KV_PAIR=0 keeps one TMA instruction per pool
    static const bool pair_allowed = [] {
        const char* v = std::getenv("MLC_B200_DECODE_KV_PAIR");
        return !(v && *v && std::atoi(v) == 0);
    }();
    const bool kv_pair = pair_allowed && a.D == 64 && pair_map_possible(a.k_pages, a.v_pages);
    if (a.ext_work) {
        // Caller-provided workspace: nothing is allocated on this path, neither on the
        // device nor (the tensor maps are encoded on the stack, uncached) on the host.
        // Each half of the caller's scratch ends with a fixed block of arrival counters for cut units, so
        // that no plan's partials - whatever its size - can ever be written where another plan's counters
        // live: the counters rely on the scratch starting zeroed and on every launch leaving them at zero.
        const size_t half = a.ext_work_bytes / 2 / 256 * 256;
        if (half <= kExtCounterBytes) return ctx->fail(MLC_ERR_UNSUPPORTED, "the fixed scratch is too small");
        const size_t partial_room = half - kExtCounterBytes;
        if (o_bytes + ml_bytes > partial_room)
            return ctx->fail(MLC_ERR_UNSUPPORTED,
                             "this batch needs %zu bytes of split-KV scratch per copy, the fixed scratch holds %zu",
                             o_bytes + ml_bytes, partial_room);
        if (static_cast<size_t>(plan.n_unit_cuts) * 4 > kExtCounterBytes)
            return ctx->fail(MLC_ERR_UNSUPPORTED,
                             "this batch cuts %u (request, head) units over CTAs, the fixed scratch has counters for %zu",
                             plan.n_unit_cuts, kExtCounterBytes / 4);
        if (kv_pair) {
            if ((st = encode_pair_map(ctx, a.k_pages, a.v_pages, a, &mk)) != MLC_OK) return st;
            mv = mk;
        } else {
            if ((st = encode_tensor_map(ctx, a.k_pages, a, &mk)) != MLC_OK) return st;
            if ((st = encode_tensor_map(ctx, a.v_pages, a, &mv)) != MLC_OK) return st;
        }
        // consecutive launches on the fixed scratch alternate between its halves, counted apart from the
        // launches on the context's own workspace
        parity = static_cast<uint32_t>(ctx->ext_launches++ & 1u);
        work = static_cast<char*>(a.ext_work) + parity * half;
        ext_counters = reinterpret_cast<uint32_t*>(work + partial_room);
        ctx->ext_counter_block[parity] = ext_counters;   // re-zeroed after a device error
    } else {
        // MLC_B200_DECODE_INKERNEL_MERGE=1: merge inside the attention kernel (arrival counters
        // [n_segs][warps], mergers poll) instead of the chained merge kernel. Measured on cfg2 it is
        // no faster (17.0 vs 16.8 us per layer on the same GPU): the chained merge kernel is already
        // resident and waiting when the attention kernel ends. Kept as an option, off by default.
        static const bool merge_kernel = [] {
            const char* v = std::getenv("MLC_B200_DECODE_INKERNEL_MERGE");
            return !(v && *v && std::atoi(v) != 0);
        }();
        use_counters = !merge_kernel && plan.n_segs > 0;
        st = ensure_workspace(ctx, 2 * (o_bytes + ml_bytes) + 512,
                              use_counters ? static_cast<size_t>(plan.n_segs) * kDecodeWarps : plan.n_unit_cuts);
        if (st != MLC_OK) return st;
        if (kv_pair) {
            if ((st = get_tensor_map(ctx, a.k_pages, a, &mk, a.v_pages)) != MLC_OK) return st;
            mv = mk;
        } else {
            if ((st = get_tensor_map(ctx, a.k_pages, a, &mk)) != MLC_OK) return st;
            if ((st = get_tensor_map(ctx, a.v_pages, a, &mv)) != MLC_OK) return st;
        }
        parity = static_cast<uint32_t>(ctx->decode_launches++ & 1u);
        work = static_cast<char*>(ctx->d_work) + parity * (ctx->work_bytes / 2 / 256 * 256);
    }

    DecodeParams prm{};
    prm.q = a.q;
    prm.o = a.o;
    prm.o_partial = a.o_partial;
    prm.ml_partial = a.ml_partial;
    prm.cta_counts = plan.cta_counts;
    prm.pieces = plan.pieces;
    prm.tile_pages = plan.tile_pages;
    prm.zero_rows = plan.zero_rows;
    prm.seg_desc = plan.seg_desc;
    prm.work_o = reinterpret_cast<float*>(work);
    prm.work_ml = reinterpret_cast<float*>(work + o_bytes);
    prm.err = ctx->d_err;
    prm.k_new = static_cast<const __half*>(a.k_new);
    prm.v_new = static_cast<const __half*>(a.v_new);
    prm.k_pool = static_cast<__half*>(const_cast<void*>(a.k_pages));
    prm.v_pool = static_cast<__half*>(const_cast<void*>(a.v_pages));
    prm.max_pieces = plan.max_pieces;
    prm.max_tiles = plan.max_tiles;
    prm.n_zero = plan.n_zero;
    prm.H = static_cast<uint32_t>(a.H);
    prm.KVH = static_cast<uint32_t>(a.KVH);
    prm.G = G;
    prm.P = static_cast<uint32_t>(a.P);
    prm.scale_log2 = a.scale * 1.4426950408889634f;
    prm.q_f32 = a.q_dtype == MLC_F32;
    prm.o_f32 = a.o_dtype == MLC_F32;
    prm.step = step ? 1 : 0;
    // Every attention launch is allowed to start early: before its wait it reads only the
    // plan (and, in a decode step, K/V rows of earlier steps).
    prm.pdl = 1;
    // Programmatic launch order is not transitive for what a kernel does before its wait: in
    // K(step s, pool A) -> K(step s, pool B) -> K(step s + 1, pool A) the third kernel may start once the
    // second has let its dependents go, while the first is still writing its new rows into pool A. Tiles
    // fetched before the wait must not come from a pool that one of the two launches before this one
    // writes, so in that case (passes of one or two layers) the early fetch is left out.
    prm.fresh_rows = (!step && a.only_plan_rows_written && plan.step_fusable) ? 1 : 0;
    prm.early_fetch = ((step || prm.fresh_rows) && recently_written(ctx, a.k_pages, a.v_pages)) ? 0 : 1;
    std::swap(ctx->recent_writes[0], ctx->recent_writes[1]);   // no allocation: the lists keep their storage
    ctx->recent_writes[1].few[0] = step ? a.k_pages : nullptr;
    ctx->recent_writes[1].few[1] = step ? a.v_pages : nullptr;
    ctx->recent_writes[1].many.clear();
    prm.stages = plan.stages;
    prm.hpc = plan.hpc ? plan.hpc : 1u;
    prm.seg_counters = use_counters ? ctx->d_counters : nullptr;
    if (plan.unit_mode && plan.n_unit_cuts) prm.seg_counters = ext_counters ? ext_counters : ctx->d_counters;
    prm.n_segs = plan.n_segs;
    {
        const uint32_t tile_bytes = static_cast<uint32_t>(kTileTokens * a.D * 2);
        const bool k_first = !kv_pair || reinterpret_cast<uintptr_t>(a.k_pages) < reinterpret_cast<uintptr_t>(a.v_pages);
        prm.kv_pair = kv_pair ? 1u : 0u;
        prm.k_off = k_first ? 0u : tile_bytes;
        prm.v_off = k_first ? tile_bytes : 0u;
    }
    // traces of consecutive launches alternate between the two halves of the buffer
    const size_t trace_need = static_cast<size_t>(plan.n_cta) * (plan.unit_mode ? unit_warps(a.D) : kDecodeWarps) * 8;
    prm.trace = ctx->d_trace && trace_need <= ctx->trace_words / 2 ? ctx->d_trace + parity * (ctx->trace_words / 2) : nullptr;
    // rows of 4 warps: a unit-mode CTA of 8 warps fills two consecutive rows
    ctx->trace_ctas = prm.trace ? plan.n_cta * (plan.unit_mode ? unit_warps(a.D) : kDecodeWarps) / kDecodeWarps : 0;
    ctx->trace_parity = parity;
    if (a.exchange) {
        // fused with the exchange across GPUs: the finished rows go to every rank, each rank combines
        const ExchangeView& xv = *a.exchange;
        PeerParams pp{};
        for (uint32_t r = 0; r < xv.world; ++r) pp.peer[r] = xv.peer[r];
        pp.local = xv.local;
        pp.out = a.exchange_out;
        pp.seq = xv.seq;
        pp.done = xv.done;
        pp.ll_off = xv.ll_off;
        pp.ll_slot_bytes = xv.ll_slot_bytes;
        pp.rank = xv.rank;
        pp.world = xv.world;
        pp.max_rows = static_cast<uint32_t>(xv.max_rows);
        pp.max_polls = ctx->wait_limit ? ctx->wait_limit : (1u << 20);
        pp.out_f32 = a.o_dtype == MLC_F32;
        prm.trace = nullptr;
        ctx->trace_ctas = 0;
        if (a.D == 64) return g16 ? launch_exchange_t<64, true>(ctx, plan, prm, mk, mv, pp) : launch_exchange_t<64, false>(ctx, plan, prm, mk, mv, pp);
        return g16 ? launch_exchange_t<128, true>(ctx, plan, prm, mk, mv, pp) : launch_exchange_t<128, false>(ctx, plan, prm, mk, mv, pp);
    }
    if (plan.unit_mode) {
        if (a.D == 64) return g16 ? launch_t<64, true, true>(ctx, plan, prm, mk, mv) : launch_t<64, false, true>(ctx, plan, prm, mk, mv);
        return g16 ? launch_t<128, true, true>(ctx, plan, prm, mk, mv) : launch_t<128, false, true>(ctx, plan, prm, mk, mv);
    }
    if (a.D == 64) return g16 ? launch_t<64, true, false>(ctx, plan, prm, mk, mv) : launch_t<64, false, false>(ctx, plan, prm, mk, mv);
    return g16 ? launch_t<128, true, false>(ctx, plan, prm, mk, mv) : launch_t<128, false, false>(ctx, plan, prm, mk, mv);
}

}  // namespace mlcb
