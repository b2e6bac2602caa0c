// A caller written against the reference's own header (compiler/runtime/metal_runtime.hpp), linked
// with include/mlc_b200_shim.cpp and libmlc_b200.so: one decode step of the batched walker's paged
// section through mlc::runtime::MetalExecutor - encodeScatterKVPagedBatched (K), the same for V,
// encodePagedFlashAttention, flush (call order of compiler/runtime/batched_walker.cpp:299-331) -
// then the synchronous variants, then the argument rules of metal_runtime.mm:7241-7243, 7742-7750.
//
//   shim_driver <in.bin> <out.bin> N H KVH D P capacity n_flat
//
// in.bin : q f32 [N,H,D] | k_new f16 [N,KVH,D] | v_new f16 | k_pool f16 [capacity,P,KVH,D] | v_pool f16 |
//          pt_flat u32 [n_flat] | pt_off u32 [N+1] | seq_lens u32 [N] | q_pos u32 [N] | page_ids u32 [N] | slots u32 [N]
// out.bin: o (encode path) f32 [N,H,D] | o (run path) f32 [N,H,D] | k_pool f16 | v_pool f16 | gathered K of request 0
//          f16 [KVH, seq_lens[0], D]
// Exit code 0 when every call behaved as the reference's contract says; the numbers are checked by the test.
//
//   shim_driver ops <in.bin> <out.bin> batch rows cols
//
// The walker's other encode* ops through the same class, weights as host vectors like the walker passes them
// (compiler/runtime/batched_walker.cpp:248-270, 340-350, 379-383):
// in.bin : x f32 [batch, cols] | norm weight f32 [cols] | W Q4_0 [rows, cols / 32 * 18] | resid f32 [batch, rows] |
//          gate_up f32 [batch, rows]   (gate = first half of a row, up = second half)
// out.bin: RMSNorm(x) f32 [batch, cols] | W * that f32 [batch, rows] | that + resid | SiLU(gate) * up f32 [batch, rows / 2]
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "runtime/metal_runtime.hpp"

using mlc::runtime::MetalExecutor;

static bool read_exact(FILE* f, void* dst, size_t bytes) { return bytes == 0 || fread(dst, 1, bytes, f) == bytes; }

#define REQUIRE(cond)                                                        \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::fprintf(stderr, "shim_driver: %s failed (line %d)\n", #cond, __LINE__); \
            return 1;                                                        \
        }                                                                    \
    } while (0)

static int run_ops(int argc, char** argv) {
    if (argc != 7) return 2;
    const size_t batch = std::strtoull(argv[4], nullptr, 10), rows = std::strtoull(argv[5], nullptr, 10);
    const size_t cols = std::strtoull(argv[6], nullptr, 10), stride = cols / 32 * 18, inner = rows / 2;
    std::vector<float> x(batch * cols), nw(cols), resid(batch * rows), gate_up(batch * rows);
    std::vector<uint8_t> w(rows * stride);
    FILE* in = std::fopen(argv[2], "rb");
    REQUIRE(in != nullptr);
    REQUIRE(read_exact(in, x.data(), x.size() * 4) && read_exact(in, nw.data(), nw.size() * 4) &&
            read_exact(in, w.data(), w.size()) && read_exact(in, resid.data(), resid.size() * 4) &&
            read_exact(in, gate_up.data(), gate_up.size() * 4));
    std::fclose(in);
    MetalExecutor& ex = MetalExecutor::Instance();
    REQUIRE(ex.isAvailable());
    void* d_x = ex.getOrAllocCachedBuffer("w_residual", x.size() * 4);
    void* d_n = ex.getOrAllocCachedBuffer("w_norm_out", x.size() * 4);
    void* d_z = ex.getOrAllocCachedBuffer("w_attn_out", resid.size() * 4);
    void* d_r = ex.getOrAllocCachedBuffer("w_resid_in", resid.size() * 4);
    void* d_a = ex.getOrAllocCachedBuffer("w_resid1", resid.size() * 4);
    void* d_gu = ex.getOrAllocCachedBuffer("w_gate_up", gate_up.size() * 4);
    void* d_g = ex.getOrAllocCachedBuffer("w_gate", batch * inner * 4);
    void* d_u = ex.getOrAllocCachedBuffer("w_up", batch * inner * 4);
    void* d_s = ex.getOrAllocCachedBuffer("w_ffn_mix", batch * inner * 4);
    REQUIRE(d_x && d_n && d_z && d_r && d_a && d_gu && d_g && d_u && d_s);
    ex.uploadToBuffer(d_x, x.data(), x.size() * 4);
    ex.uploadToBuffer(d_r, resid.data(), resid.size() * 4);
    ex.uploadToBuffer(d_gu, gate_up.data(), gate_up.size() * 4);
    REQUIRE(!ex.encodeRmsNormBatched(d_x, nw, 1e-5f, batch, cols, d_n));   // no open pass
    REQUIRE(ex.beginForwardPassCB());
    REQUIRE(ex.encodeRmsNormBatched(d_x, nw, 1e-5f, batch, cols, d_n));
    REQUIRE(ex.encodeMatMulQ4_0Batched("blk.0.attn_output.weight", w, d_n, batch, rows, cols, stride, 2, d_z));
    REQUIRE(ex.encodeAddBatched(d_z, d_r, d_a, batch * rows));
    REQUIRE(ex.encodeGateUpSplitSiluMul(d_gu, d_g, d_u, d_s, batch, inner, rows));
    // a second call with the same weight name reuses the device copy (getOrCacheWeight, metal_runtime.mm:3715)
    REQUIRE(ex.encodeMatMulQ4_0Batched("blk.0.attn_output.weight", w, d_n, batch, rows, cols, stride, 2, d_z));
    REQUIRE(ex.flushForwardPassCB());
    std::vector<float> n(x.size()), z(resid.size()), a(resid.size()), sm(batch * inner);
    ex.downloadFromBuffer(d_n, n.data(), n.size() * 4);
    ex.downloadFromBuffer(d_z, z.data(), z.size() * 4);
    ex.downloadFromBuffer(d_a, a.data(), a.size() * 4);
    ex.downloadFromBuffer(d_s, sm.data(), sm.size() * 4);
    FILE* out = std::fopen(argv[3], "wb");
    REQUIRE(out != nullptr);
    std::fwrite(n.data(), 4, n.size(), out);
    std::fwrite(z.data(), 4, z.size(), out);
    std::fwrite(a.data(), 4, a.size(), out);
    std::fwrite(sm.data(), 4, sm.size(), out);
    std::fclose(out);
    std::puts("shim_driver: ok");
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 2 && std::string(argv[1]) == "ops") return run_ops(argc, argv);
    if (argc != 10) {
        std::fprintf(stderr, "usage: shim_driver in out N H KVH D P capacity n_flat\n");
        return 2;
    }
    const size_t N = std::strtoull(argv[3], nullptr, 10), H = std::strtoull(argv[4], nullptr, 10);
    const size_t KVH = std::strtoull(argv[5], nullptr, 10), D = std::strtoull(argv[6], nullptr, 10);
    const size_t P = std::strtoull(argv[7], nullptr, 10), capacity = std::strtoull(argv[8], nullptr, 10);
    const size_t n_flat = std::strtoull(argv[9], nullptr, 10);
    const size_t q_elems = N * H * D, row_elems = N * KVH * D, pool_elems = capacity * P * KVH * D;

    std::vector<float> q(q_elems);
    std::vector<uint16_t> k_new(row_elems), v_new(row_elems), k_pool(pool_elems), v_pool(pool_elems);
    std::vector<uint32_t> pt_flat(n_flat), pt_off(N + 1), seq_lens(N), q_pos(N), page_ids(N), slots(N);
    FILE* in = std::fopen(argv[1], "rb");
    REQUIRE(in != nullptr);
    REQUIRE(read_exact(in, q.data(), q_elems * 4) && read_exact(in, k_new.data(), row_elems * 2) &&
            read_exact(in, v_new.data(), row_elems * 2) && read_exact(in, k_pool.data(), pool_elems * 2) &&
            read_exact(in, v_pool.data(), pool_elems * 2) && read_exact(in, pt_flat.data(), n_flat * 4) &&
            read_exact(in, pt_off.data(), (N + 1) * 4) && read_exact(in, seq_lens.data(), N * 4) &&
            read_exact(in, q_pos.data(), N * 4) && read_exact(in, page_ids.data(), N * 4) &&
            read_exact(in, slots.data(), N * 4));
    std::fclose(in);

    MetalExecutor& ex = MetalExecutor::Instance();
    REQUIRE(ex.isAvailable());
    void* d_q = ex.allocateScratchBuffer(q_elems * 4);
    void* d_o = ex.allocateScratchBuffer(q_elems * 4);
    void* d_o2 = ex.allocateScratchBuffer(q_elems * 4);
    void* d_kn = ex.allocateScratchBuffer(row_elems * 2);
    void* d_vn = ex.allocateScratchBuffer(row_elems * 2);
    void* d_kp = ex.allocateScratchBuffer(pool_elems * 2);
    void* d_vp = ex.allocateScratchBuffer(pool_elems * 2);
    void* d_kp2 = ex.allocateScratchBuffer(pool_elems * 2);
    void* d_vp2 = ex.allocateScratchBuffer(pool_elems * 2);
    REQUIRE(d_q && d_o && d_o2 && d_kn && d_vn && d_kp && d_vp && d_kp2 && d_vp2);
    ex.uploadToBuffer(d_q, q.data(), q_elems * 4);
    ex.uploadToBuffer(d_kn, k_new.data(), row_elems * 2);
    ex.uploadToBuffer(d_vn, v_new.data(), row_elems * 2);
    ex.uploadToBuffer(d_kp, k_pool.data(), pool_elems * 2);
    ex.uploadToBuffer(d_vp, v_pool.data(), pool_elems * 2);
    ex.uploadToBuffer(d_kp2, k_pool.data(), pool_elems * 2);
    ex.uploadToBuffer(d_vp2, v_pool.data(), pool_elems * 2);

    // ---- the walker's order on one pass: nothing may be encoded without an open pass (metal_runtime.mm:7090)
    REQUIRE(!ex.hasForwardPassCB());
    REQUIRE(!ex.encodeScatterKVPagedBatched(d_kp, page_ids, slots, P, KVH, D, N, d_kn));
    REQUIRE(ex.beginForwardPassCB());
    REQUIRE(ex.hasForwardPassCB());
    REQUIRE(ex.encodeScatterKVPagedBatched(d_kp, page_ids, slots, P, KVH, D, N, d_kn));
    REQUIRE(ex.encodeScatterKVPagedBatched(d_vp, page_ids, slots, P, KVH, D, N, d_vn));
    REQUIRE(ex.encodePagedFlashAttention(d_q, d_kp, d_vp, d_o, pt_flat, pt_off, seq_lens, q_pos, N, H, KVH, D, P, true));
    REQUIRE(ex.flushForwardPassCB());
    REQUIRE(!ex.hasForwardPassCB());

    // ---- the synchronous variants on a second copy of the pools
    REQUIRE(ex.scatterKVPagedBatched(d_kp2, page_ids, slots, P, KVH, D, N, d_kn));
    REQUIRE(ex.scatterKVPagedBatched(d_vp2, page_ids, slots, P, KVH, D, N, d_vn));
    REQUIRE(ex.runPagedFlashAttention(d_q, d_kp2, d_vp2, d_o2, pt_flat, pt_off, seq_lens, q_pos, N, H, KVH, D, P, true));

    // ---- gather of request 0's K rows, [KVH, S, D]
    const size_t S0 = seq_lens[0];
    std::vector<uint32_t> table0(pt_flat.begin() + pt_off[0], pt_flat.begin() + pt_off[1]);
    void* d_g = ex.allocateScratchBuffer(KVH * S0 * D * 2 + 16);
    REQUIRE(d_g != nullptr);
    REQUIRE(ex.gatherKVPages(d_kp, table0, P, KVH, D, S0, d_g, 2));

    // ---- argument rules (each must come back false and leave everything usable)
    std::vector<uint32_t> short_ids(page_ids.begin(), page_ids.end() - (N > 1 ? 1 : 0));
    if (N > 1) REQUIRE(!ex.scatterKVPagedBatched(d_kp2, short_ids, slots, P, KVH, D, N, d_kn));
    REQUIRE(!ex.scatterKVPagedBatched(nullptr, page_ids, slots, P, KVH, D, N, d_kn));
    REQUIRE(!ex.scatterKVPagedBatched(d_kp2, page_ids, slots, 0, KVH, D, N, d_kn));
    std::vector<uint32_t> bad_off(pt_off.begin(), pt_off.end() - 1);
    REQUIRE(!ex.runPagedFlashAttention(d_q, d_kp2, d_vp2, d_o2, pt_flat, bad_off, seq_lens, q_pos, N, H, KVH, D, P, true));
    REQUIRE(!ex.runPagedFlashAttention(d_q, d_kp2, d_vp2, d_o2, pt_flat, pt_off, seq_lens, q_pos, N, H, 3, D, P, true));
    REQUIRE(!ex.runPagedFlashAttention(nullptr, d_kp2, d_vp2, d_o2, pt_flat, pt_off, seq_lens, q_pos, N, H, KVH, D, P, true));
    REQUIRE(!ex.gatherKVPages(d_kp, table0, P, KVH, D, S0, d_g, 3));
    REQUIRE(!ex.scatterKVPaged(d_kp2, table0, P, KVH, D, 1, P, d_kn, 2));   // start_slot >= page size

    std::vector<float> o(q_elems), o2(q_elems);
    std::vector<uint16_t> g(KVH * S0 * D);
    ex.downloadFromBuffer(d_o, o.data(), q_elems * 4);
    ex.downloadFromBuffer(d_o2, o2.data(), q_elems * 4);
    ex.downloadFromBuffer(d_kp, k_pool.data(), pool_elems * 2);
    ex.downloadFromBuffer(d_vp, v_pool.data(), pool_elems * 2);
    ex.downloadFromBuffer(d_g, g.data(), g.size() * 2);
    FILE* out = std::fopen(argv[2], "wb");
    REQUIRE(out != nullptr);
    std::fwrite(o.data(), 4, q_elems, out);
    std::fwrite(o2.data(), 4, q_elems, out);
    std::fwrite(k_pool.data(), 2, pool_elems, out);
    std::fwrite(v_pool.data(), 2, pool_elems, out);
    std::fwrite(g.data(), 2, g.size(), out);
    std::fclose(out);
    for (void* b : {d_q, d_o, d_o2, d_kn, d_vn, d_kp, d_vp, d_kp2, d_vp2, d_g}) ex.releaseScratchBuffer(b);
    std::puts("shim_driver: ok");
    return 0;
}
