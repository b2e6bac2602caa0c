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
#include <cstdint>
#include <cstdio>
#include <cstdlib>
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

int main(int argc, char** argv) {
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
