// Chunked (multi-token) causal paged attention on the 5th-generation tensor cores:
// tcgen05.mma with accumulators in tensor memory (TMEM), operands staged by TMA.
//
// The reference has no multi-token paged kernel: with paged storage its prefill is a loop
// of single-token decode passes (compiler/runtime/batched_executor.cpp:450-467), and its
// CPU backend defines multi-token attention as that same loop
// (compiler/runtime/operator_backend.cpp:906-968): query i of a request sits at position
// q_start + i and sees kv_pos <= q_start + i (mask rule metal_runtime.mm:2286). This
// kernel computes exactly that for all query tokens at once - a dense contraction, which
// is why it, unlike the decode kernel, belongs on tcgen05.
//
// One CTA = 128 query tokens of one (request, query head). Per 64-token page of K/V:
//   S[128x64]  = Q[128x128] . K^T           tcgen05.mma kind::f16, A and B from shared memory
//                                           (K-major, 128-byte swizzle), fp32 accumulator in TMEM
//   softmax    : thread t owns row t: tcgen05.ld its 64 scores, mask, running max / sum in fp32
//                (base-2 exponentials), P rounded to fp16 and stored back into tensor memory over its
//                own scores (tcgen05.st) as the next A operand - P never touches shared memory, whose
//                bandwidth is what bounds this kernel; the O accumulator is rescaled only when a row's maximum
//                has grown by more than 2^8 since the last rescale (exact: the final 1/l uses the
//                same reference maximum)
//   O[128x128] += P[128x64] . V[64x128]     tcgen05.mma, A = P from TMEM, B = V tile as an MN-major operand
// Warps 0-3: softmax / epilogue (warp w reads TMEM lanes 32w..32w+31), warp 4: MMA issue
// (one elected lane) and TMEM allocation, warps 5 / 6: TMA producers of K / V. S is double-buffered in
// TMEM so Q.K^T of page j+1 runs under the softmax of page j. No cluster, no multicast.
// Every mbarrier wait is bounded; on expiry the CTA records MLC_DEVERR_WAIT_TIMEOUT,
// frees its TMEM and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstring>

#include "attn_internal.hpp"

namespace mlcb {

namespace {

constexpr int kQTile = 128;      // query rows per CTA (= TMEM lanes)
constexpr int kKvTile = 64;      // tokens per K/V tile (= one page)
constexpr int kHeadDim = 128;
constexpr int kStages = 2;
constexpr uint32_t kSubBytesQ = kQTile * 128;    // one 64-half-wide slab of the Q tile
constexpr uint32_t kSubBytesKV = kKvTile * 128;  // one 64-half-wide slab of a K or V tile
constexpr uint32_t kQBytes = 2 * kSubBytesQ;     // 32 KiB
constexpr uint32_t kKvBytes = 2 * kSubBytesKV;   // 16 KiB per tensor
constexpr uint32_t kTileBytes = kQBytes + kStages * 2 * kKvBytes;  // 96 KiB
struct Bars {
    uint64_t q, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages], s_full[2], p_full[2], pv_done;
    uint32_t tmem_slot;
};
constexpr uint32_t kSmemBytes = kTileBytes + sizeof(Bars);
constexpr uint32_t kTmemCols = 256;              // O: 128 columns, S: 2 x 64 columns
constexpr uint32_t kTmemO = 0, kTmemS = 128;

struct PrefillParams {
    void* o;                        // fp16 [sum q_len, H, D]
    const uint32_t* pt_flat;
    const uint32_t* pt_off;
    const uint32_t* seq_lens;
    const uint32_t* q_start;
    const uint32_t* q_len;
    const uint32_t* q_row0;         // first row of each request in q / o
    uint32_t* err;
    uint32_t H, KVH, G;
    float scale_log2;
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    // a poll that finds the phase open suspends for a few microseconds: 2^18 polls are about a second
    for (uint32_t i = 0; i < (1u << 18); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- tcgen05 wrappers ----------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem], kind::f16 (fp16 operands, fp32 accumulate)
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Same with the A operand read from tensor memory: lane = row, one 32-bit column = two
// consecutive fp16 elements along K.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte
// offsets in 16-byte units, descriptor version 1 (bit 46), layout type 2 (bits 61-63).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor of kind::f16: fp32 accumulator, fp16 A and B, A K-major,
// B K-major (b_mn_major = 0) or MN-major (1), shape M x N.
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t M, uint32_t N, uint32_t b_mn_major) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (b_mn_major << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

}  // namespace

__global__ void __launch_bounds__(224, 2)
paged_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                             const __grid_constant__ CUtensorMap tmV, const PrefillParams prm) {
    // All shared memory is dynamic (tiles first, barriers behind them) so that two CTAs fit one SM.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Bars& bars = *reinterpret_cast<Bars*>(smem_raw + kTileBytes);
    uint64_t& bar_q = bars.q;
    uint64_t(&bar_k_full)[kStages] = bars.k_full;
    uint64_t(&bar_k_empty)[kStages] = bars.k_empty;
    uint64_t(&bar_v_full)[kStages] = bars.v_full;
    uint64_t(&bar_v_empty)[kStages] = bars.v_empty;
    uint64_t(&bar_s_full)[2] = bars.s_full;
    uint64_t(&bar_p_full)[2] = bars.p_full;
    uint64_t& bar_pv_done = bars.pv_done;
    uint32_t& tmem_base_slot = bars.tmem_slot;

    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
    // the last query tile of a chunk sees the most keys: launch the long CTAs first
    const uint32_t req = blockIdx.z, head = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;
    const uint32_t q_len = prm.q_len[req];
    if (qt * kQTile >= q_len) return;  // uniform over the CTA, before any barrier or TMEM use
    const uint32_t q_start = prm.q_start[req];
    const uint32_t seq_len = prm.seq_lens[req];
    const uint32_t q_row0 = prm.q_row0[req] + qt * kQTile;            // first row of this tile in q / o
    const uint32_t q_rows = min(static_cast<uint32_t>(kQTile), q_len - qt * kQTile);
    const uint32_t kv_head = static_cast<uint32_t>((static_cast<uint64_t>(head) * prm.KVH) / prm.H);
    // last position any row of this tile may look at, exclusive
    const uint32_t kv_end = min(seq_len, q_start + qt * kQTile + q_rows);
    const uint32_t n_tiles = (kv_end + kKvTile - 1) / kKvTile;

    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {  // the 128-byte swizzle needs 1024-byte aligned tiles; never expected
        if (threadIdx.x == 0) atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT | (0x40u << 8));
        return;
    }
    const uint32_t sQ = base;
    const uint32_t sKV = sQ + kQBytes;                       // stage s: K at sKV + s*2*kKvBytes, V right after K

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar_q), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_k_full[s]), 1);
            mbar_init(smem_u32(&bar_k_empty[s]), 1);
            mbar_init(smem_u32(&bar_v_full[s]), 1);
            mbar_init(smem_u32(&bar_v_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_s_full[b]), 1);
            // Two P barriers, like the two S buffers: the softmax warps may finish page j+1 (its
            // scores were issued early) before the MMA warp has looked at page j's arrival; with one
            // barrier that second completion would flip the phase parity back and the wait would
            // never see page j.
            mbar_init(smem_u32(&bar_p_full[b]), 128);
        }
        mbar_init(smem_u32(&bar_pv_done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;

    // A wait that ran out records the timeout bit plus where it gave up: bits 8-15 = which wait
    // (0x1x MMA warp, 0x2x softmax, 0x3x producers), bits 16-31 = the page it was working on.
    auto give_up = [&](uint32_t where, uint32_t tile) {
        // the first failure's detail wins; later ones only (re)set the timeout bit
        if (lane == 0 && atomicCAS(prm.err, 0u, MLC_DEVERR_WAIT_TIMEOUT | (where << 8) | (tile << 16)) != 0u)
            atomicOr(prm.err, MLC_DEVERR_WAIT_TIMEOUT);
    };

    if (warp == 5) {
        // ---------------- TMA producer of Q and the K tiles ----------------
        // A K stage is free again as soon as the Q.K^T that read it has completed, a V stage
        // only after its P.V: the two streams have their own barriers and their own warp.
        if (lane == 0 && n_tiles > 0) {
            const uint32_t bq = smem_u32(&bar_q);
            mbar_expect_tx(bq, kQBytes);
            tma_load_3d(sQ, &tmQ, bq, 0, static_cast<int>(head), static_cast<int>(q_row0));
            tma_load_3d(sQ + kSubBytesQ, &tmQ, bq, 64, static_cast<int>(head), static_cast<int>(q_row0));
            const uint32_t pt_base = prm.pt_off[req];
            for (uint32_t j = 0; j < n_tiles; ++j) {
                const uint32_t s = j % kStages;
                if (j >= kStages && !mbar_wait_bounded(smem_u32(&bar_k_empty[s]), ((j / kStages) - 1) & 1u)) {
                    give_up(0x30, j);
                    break;
                }
                const int page = static_cast<int>(prm.pt_flat[pt_base + j]);
                const uint32_t bf = smem_u32(&bar_k_full[s]);
                const uint32_t dK = sKV + s * 2 * kKvBytes;
                mbar_expect_tx(bf, kKvBytes);
                tma_load_4d(dK, &tmK, bf, 0, static_cast<int>(kv_head), 0, page);
                tma_load_4d(dK + kSubBytesKV, &tmK, bf, 64, static_cast<int>(kv_head), 0, page);
            }
        }
    } else if (warp == 6) {
        // ---------------- TMA producer of the V tiles ----------------
        if (lane == 0 && n_tiles > 0) {
            const uint32_t pt_base = prm.pt_off[req];
            for (uint32_t j = 0; j < n_tiles; ++j) {
                const uint32_t s = j % kStages;
                if (j >= kStages && !mbar_wait_bounded(smem_u32(&bar_v_empty[s]), ((j / kStages) - 1) & 1u)) {
                    give_up(0x31, j);
                    break;
                }
                const int page = static_cast<int>(prm.pt_flat[pt_base + j]);
                const uint32_t bf = smem_u32(&bar_v_full[s]);
                const uint32_t dV = sKV + s * 2 * kKvBytes + kKvBytes;
                mbar_expect_tx(bf, kKvBytes);
                tma_load_4d(dV, &tmV, bf, 0, static_cast<int>(kv_head), 0, page);
                tma_load_4d(dV + kSubBytesKV, &tmV, bf, 64, static_cast<int>(kv_head), 0, page);
            }
        }
    } else if (warp == 4) {
        // ---------------- MMA issue ----------------
        // The whole warp walks the loop (waits, addresses and descriptors stay warp-uniform, so the
        // compiler can keep them in uniform registers); one elected lane issues the instructions.
        if (n_tiles > 0) {
            constexpr uint32_t idesc_qk = idesc_f16(kQTile, kKvTile, 0);    // S = Q.K^T : B = K tile, K-major
            constexpr uint32_t idesc_pv = idesc_f16(kQTile, kHeadDim, 1);   // O += P.V  : B = V tile, MN-major
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
            const uint32_t sQ_u = __shfl_sync(0xffffffffu, sQ, 0);
            const uint64_t desc_k_major = smem_desc_sw128(0, 16, 1024);
            const uint64_t desc_v = smem_desc_sw128(0, kSubBytesKV, 1024);
            auto issue_qk = [&](uint32_t j) {
                const uint32_t s = j % kStages;
                const uint32_t sK = sQ_u + kQBytes + s * 2 * kKvBytes;
                const uint32_t d = tmem_u + kTmemS + (j & 1u) * kKvTile;
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < kHeadDim / 16; ++k) {  // 16 halfs = 32 bytes per step inside a 128-byte row
                        const uint32_t a = sQ_u + (k >> 2) * kSubBytesQ + (k & 3) * 32;
                        const uint32_t b = sK + (k >> 2) * kSubBytesKV + (k & 3) * 32;
                        tc_mma_f16(d, desc_k_major | (a >> 4), desc_k_major | (b >> 4), idesc_qk, k > 0);
                    }
                    tc_commit(smem_u32(&bar_k_empty[s]));
                    tc_commit(smem_u32(&bar_s_full[j & 1u]));
                }
                __syncwarp();
            };
            uint32_t where = 0x10, at = 0;
            bool ok = mbar_wait_bounded(smem_u32(&bar_q), 0) && mbar_wait_bounded(smem_u32(&bar_k_full[0]), 0);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after();
                issue_qk(0);
            }
            for (uint32_t j = 0; ok && j < n_tiles; ++j) {
                at = j;
                if (j + 1 < n_tiles) {  // Q.K^T of the next page runs under this page's softmax
                    const uint32_t s1 = (j + 1) % kStages;
                    where = 0x11;
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_k_full[s1]), ((j + 1) / kStages) & 1u));
                    // S buffer (j+1)&1 still holds P of page j-1 (P overwrites S in place): its P.V must be done
                    if (ok && j >= 1) {
                        where = 0x12;
                        ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_pv_done), (j - 1) & 1u));
                    }
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1);
                }
                const uint32_t s = j % kStages;
                where = 0x13;
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_v_full[s]), (j / kStages) & 1u));
                if (ok) {
                    where = 0x14;
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&bar_p_full[j & 1u]), (j >> 1) & 1u));
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t sV = sQ_u + kQBytes + s * 2 * kKvBytes + kKvBytes;
                const uint32_t pj = tmem_u + kTmemS + (j & 1u) * kKvTile;
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < kKvTile / 16; ++k) {  // 16 tokens per step
                        const uint32_t b = sV + k * 16 * 128;  // V: 16 token rows further down
                        // P in TMEM: 16 fp16 = 8 columns per step
                        tc_mma_f16_ts(tmem_u + kTmemO, pj + k * 8, desc_v | (b >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&bar_v_empty[s]));
                    tc_commit(smem_u32(&bar_pv_done));
                }
                __syncwarp();
            }
            if (!ok) give_up(where, at);
        }
    } else {
        // ---------------- softmax + epilogue: thread = query row ----------------
        const uint32_t row = threadIdx.x;                      // 0..127 = TMEM lane
        const uint32_t lane_base = (warp * 32u) << 16;
        const uint32_t q_pos = q_start + qt * kQTile + row;    // position of this row's query token
        const uint32_t q_pos_warp = q_start + qt * kQTile + warp * 32u;  // smallest position in this warp
        const float rescale_step = 8.0f / prm.scale_log2;      // 2^8 in units of the unscaled scores
        float m_ref = -INFINITY, l_sum = 0.f;                  // reference maximum of the O accumulator, row sum
        bool ok = true;
        uint32_t where = 0x20, at = 0;
        for (uint32_t j = 0; j < n_tiles; ++j) {
            at = j;
            where = 0x20;
            ok = ok && mbar_wait_bounded(smem_u32(&bar_s_full[j & 1u]), (j >> 1) & 1u);
            if (!ok) break;
            tc_fence_after();
            uint32_t sreg[64];
            {
                uint32_t lo[32], hi[32];
                tmem_ld32(tmem + lane_base + kTmemS + (j & 1u) * kKvTile, lo);
                tmem_ld32(tmem + lane_base + kTmemS + (j & 1u) * kKvTile + 32, hi);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) { sreg[i] = lo[i]; sreg[32 + i] = hi[i]; }
            }
            // mask: causal (kv_pos > q_pos) and past the end of the sequence
            const uint32_t kv0 = j * kKvTile;
            // Scores stay unscaled (scale > 0 keeps their order); the scale is folded into the
            // exponent's FMA below. Only a tile that crosses the diagonal of some row of this
            // warp, or the end of the sequence, pays for the mask (warp-uniform test).
            if (kv0 + kKvTile - 1 > q_pos_warp || kv0 + kKvTile > seq_len) {
                const uint32_t lim = min(q_pos + 1, seq_len);  // first masked position
#pragma unroll
                for (int c = 0; c < kKvTile; ++c)
                    if (kv0 + c >= lim) sreg[c] = 0xff800000u;  // -inf
            }
            float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < kKvTile; c += 4) {
                t0 = fmaxf(t0, __uint_as_float(sreg[c]));
                t1 = fmaxf(t1, __uint_as_float(sreg[c + 1]));
                t2 = fmaxf(t2, __uint_as_float(sreg[c + 2]));
                t3 = fmaxf(t3, __uint_as_float(sreg[c + 3]));
            }
            const float m_new = fmaxf(m_ref, fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)));
            // Rescale O only when this row's maximum outgrew the reference by more than 2^8
            // (P stays <= 256 otherwise, well inside fp16). The vote keeps the warp together:
            // tcgen05.ld / .st are warp-wide.
            const bool need = (m_new > m_ref + rescale_step) || (m_ref == -INFINITY && m_new > -INFINITY);
            const float alpha = need ? ((m_ref == -INFINITY) ? 0.f : ex2((m_ref - m_new) * prm.scale_log2)) : 1.0f;
            if (need) m_ref = m_new;
            l_sum *= alpha;
            // P = exp2((s - m_ref) * scale), fp16, computed while the previous P.V may still run, then
            // stored into the swizzled A-operand tile: row `row`, 8 chunks of 16 bytes
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * prm.scale_log2;
            float ps[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float p0 = ex2(fmaf(__uint_as_float(sreg[ch * 8 + 2 * i]), prm.scale_log2, neg_m));
                    const float p1 = ex2(fmaf(__uint_as_float(sreg[ch * 8 + 2 * i + 1]), prm.scale_log2, neg_m));
                    ps[i] += p0 + p1;
                    __half2 h = __floats2half2_rn(p0, p1);
                    w[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                pk[ch * 4 + 0] = w[0]; pk[ch * 4 + 1] = w[1]; pk[ch * 4 + 2] = w[2]; pk[ch * 4 + 3] = w[3];
            }
            l_sum += (ps[0] + ps[1]) + (ps[2] + ps[3]);
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                // O may only be touched once the previous P.V is done (warp-uniform branch)
                where = 0x21;
                ok = mbar_wait_bounded(smem_u32(&bar_pv_done), (j - 1) & 1u);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                    uint32_t oreg[32];
                    tmem_ld32(tmem + lane_base + kTmemO + c0, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                    tmem_st32(tmem + lane_base + kTmemO + c0, oreg);
                }
                tmem_wait_st();
            }
            // P overwrites the first 32 columns of this page's S buffer (own lane only, already read)
            tmem_st32(tmem + lane_base + kTmemS + (j & 1u) * kKvTile, pk);
            tmem_wait_st();
            // V rows past the end of the sequence may hold anything: zero them (last page only)
            if (kv0 + kKvTile > seq_len) {
                where = 0x22;
                ok = mbar_wait_bounded(smem_u32(&bar_v_full[j % kStages]), (j / kStages) & 1u);  // the tile has landed
                if (!ok) break;
                const uint32_t sV = sKV + (j % kStages) * 2 * kKvBytes + kKvBytes;
                const uint32_t first = seq_len - kv0;  // 1..63
                for (uint32_t i = threadIdx.x; i < (kKvTile - first) * 16; i += 128) {
                    const uint32_t r = first + (i >> 4), c = i & 15;
                    const uint32_t addr = sV + (c >> 3) * kSubBytesKV + r * 128 + ((c & 7) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            // Every warp follows bar_pv_done phase by phase: a parity wait tells "phase k done" from "phase k - 2
            // done" only for a waiter that is at most one phase behind, and a warp that only waited when it had to
            // rescale O could reach the epilogue's wait two phases behind (the last page's scores are issued
            // early, so its softmax can finish while P.V of the page before still runs) and read O too soon.
            // Waiting here costs nothing: P.V of this page cannot start before the one before it has finished,
            // and it cannot have been issued yet (this warp has not arrived), so the barrier is 0 or 1 phases on.
            if (j > 0) {
                where = 0x24;
                ok = mbar_wait_bounded(smem_u32(&bar_pv_done), (j - 1) & 1u);
                if (!ok) break;
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_p_full[j & 1u]));
        }
        if (ok && n_tiles > 0) {
            // the last P.V must be complete before O is read (this warp has seen every earlier phase, see above)
            where = 0x23;
            ok = mbar_wait_bounded(smem_u32(&bar_pv_done), (n_tiles - 1) & 1u);
        }
        if (!ok) {
            give_up(where, at);
        } else {
            tc_fence_after();
            const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
            __half* dst = static_cast<__half*>(prm.o) + (static_cast<size_t>(q_row0 + row) * prm.H + head) * kHeadDim;
#pragma unroll 1
            for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
                uint32_t oreg[32];
                if (n_tiles > 0) {
                    tmem_ld32(tmem + lane_base + kTmemO + c0, oreg);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) oreg[i] = 0u;
                }
                if (row < q_rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 pk;
                        __half2 h0 = __floats2half2_rn(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv);
                        __half2 h1 = __floats2half2_rn(__uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv);
                        __half2 h2 = __floats2half2_rn(__uint_as_float(oreg[i + 4]) * inv, __uint_as_float(oreg[i + 5]) * inv);
                        __half2 h3 = __floats2half2_rn(__uint_as_float(oreg[i + 6]) * inv, __uint_as_float(oreg[i + 7]) * inv);
                        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(dst + c0 + i) = pk;
                    }
                }
            }
        }
    }
    // ---------------- teardown: every tcgen05 operation is finished, free the TMEM columns ----------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 4) tmem_dealloc(tmem, kTmemCols);
}

// --------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_map(mlc_ctx* ctx, CUtensorMap* out, const void* ptr, uint32_t rank, const cuuint64_t* dims,
                      const cuuint64_t* strides, const cuuint32_t* box) {
    if (!ctx->tmap_encode_fn) {
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->tmap_encode_fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !ctx->tmap_encode_fn)
            return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    }
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->tmap_encode_fn)(
        out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ctx->fail(MLC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return MLC_OK;
}

bool prefill_tcgen05_supported(size_t H, size_t KVH, size_t D, size_t P, size_t capacity) {
    return D == kHeadDim && P == kKvTile && KVH > 0 && H % KVH == 0 && capacity > 0;
}

int launch_prefill_tcgen05(mlc_ctx* ctx, const void* q, const void* k_pages, const void* v_pages, void* o,
                           const uint32_t* d_pt_flat, const uint32_t* d_pt_off, const uint32_t* d_seq_lens,
                           const uint32_t* d_q_start, const uint32_t* d_q_len, const uint32_t* d_q_row0,
                           size_t batch, size_t total_q, size_t max_q_len, size_t H, size_t KVH, size_t capacity,
                           float scale) {
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {kHeadDim, H, total_q};
        cuuint64_t strides[2] = {kHeadDim * 2, H * kHeadDim * 2};
        cuuint32_t box[3] = {64, 1, kQTile};
        int st = encode_map(ctx, &mq, q, 3, dims, strides, box);
        if (st != MLC_OK) return st;
    }
    {
        cuuint64_t dims[4] = {kHeadDim, KVH, kKvTile, capacity};
        cuuint64_t strides[3] = {kHeadDim * 2, KVH * kHeadDim * 2, static_cast<cuuint64_t>(kKvTile) * KVH * kHeadDim * 2};
        cuuint32_t box[4] = {64, 1, kKvTile, 1};
        int st = encode_map(ctx, &mk, k_pages, 4, dims, strides, box);
        if (st == MLC_OK) st = encode_map(ctx, &mv, v_pages, 4, dims, strides, box);
        if (st != MLC_OK) return st;
    }
    if (!ctx->prefill_smem_set) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(paged_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(kSmemBytes)));
        ctx->prefill_smem_set = true;
    }
    PrefillParams prm{};
    prm.o = o;
    prm.pt_flat = d_pt_flat;
    prm.pt_off = d_pt_off;
    prm.seq_lens = d_seq_lens;
    prm.q_start = d_q_start;
    prm.q_len = d_q_len;
    prm.q_row0 = d_q_row0;
    prm.err = ctx->d_err;
    prm.H = static_cast<uint32_t>(H);
    prm.KVH = static_cast<uint32_t>(KVH);
    prm.G = static_cast<uint32_t>(H / KVH);
    prm.scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(static_cast<unsigned>((max_q_len + kQTile - 1) / kQTile), static_cast<unsigned>(H), static_cast<unsigned>(batch));
    paged_prefill_tcgen05_kernel<<<grid, 224, kSmemBytes, ctx->stream>>>(mq, mk, mv, prm);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

}  // namespace mlcb
