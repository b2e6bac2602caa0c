/*
 * CPU restatement of MLcompiler's paged-attention hot path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA kernels are
 * compared against. Only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may build, load or call it; the product library never does.
 *
 * Parity pins (all exercised by the CPU test-suite):
 *   - the reference's own executor-CPU attention (RunAttentionCPU,
 *     compiler/runtime/attention_cpu.cpp:272-478) linked from its unmodified
 *     sources, on identical seeded inputs;
 *   - the known-answer vectors of compiler/main.cpp:4026-4031 (tiny case) and
 *     tests/test_runtime.cpp:1691-1716, the stress-online construction of
 *     compiler/main.cpp:4033-4065, the scatter/gather patterns of
 *     tests/test_paged_kv.cpp:219-267,404-474 and the allocator sequences of
 *     tests/test_paged_kv.cpp:34-207.
 *
 * Each function names the reference lines it follows. Index arithmetic is
 * 64-bit here (the reference's is 32-bit, compiler/runtime/metal_runtime.mm:2271);
 * for every pool smaller than 2^32 elements the two agree exactly.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------ */
/* fp16 bit conventions: compiler/runtime/float_convert.hpp:14-76            */
/* ------------------------------------------------------------------------ */

/* float_convert.hpp:14-48 (normal, subnormal, inf/nan cases). */
float orc_fp16_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t hexp = h & 0x7C00u, hsig = h & 0x03FFu, exp, man;
    if (hexp == 0) {
        if (hsig == 0) {
            exp = 0; man = 0;
        } else {
            uint32_t shift = 0;
            while ((hsig & 0x0400u) == 0) { hsig <<= 1; ++shift; }
            hsig &= 0x03FFu;
            man = hsig << 13;
            exp = 127 - 14 - shift;
        }
    } else if (hexp == 0x7C00u) {
        exp = 255; man = hsig << 13;
    } else {
        exp = (hexp >> 10) - 15 + 127; man = hsig << 13;
    }
    uint32_t w = sign | (exp << 23) | man;
    float f; memcpy(&f, &w, 4);
    return f;
}

/* float_convert.hpp:57-76: the reference's scalar encoder. It rounds by adding
 * 0x1000 before the shift (ties away from zero), flushes below 2^-25 to zero
 * and maps NaN to infinity. */
uint16_t orc_float_to_fp16_ref_scalar(float v) {
    uint32_t bits; memcpy(&bits, &v, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t exp = (int32_t)((bits >> 23) & 0xFF) - 127 + 15;
    uint32_t man = bits & 0x7FFFFFu;
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man = (man | 0x800000u) >> (1 - exp);
        return (uint16_t)(sign | ((man + 0x1000u) >> 13));
    }
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)exp << 10) | ((man + 0x1000u) >> 13));
}

/* Round-to-nearest-even encoder: what Metal's half(x) (metal_runtime.mm:465) and
 * the reference's NEON path (float_convert.hpp:96-101) produce. */
uint16_t orc_float_to_fp16_rne(float v) {
    uint32_t x; memcpy(&x, &v, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);          /* rounds to inf */
    if (x < 0x33000001u) return (uint16_t)sign;                        /* <= 2^-25 */
    int32_t e = (int32_t)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    uint32_t shift = (e < -14) ? (uint32_t)(13 + (-14 - e)) : 13u;
    uint32_t half_m = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_m & 1))) ++half_m;
    uint32_t he = (e < -14) ? 0u : (uint32_t)(e + 15);
    /* half_m carries the implicit bit for normals; adding lets a mantissa carry
     * bump the exponent. */
    uint32_t out = (e < -14) ? half_m : ((he << 10) + (half_m - 0x400u));
    return (uint16_t)(sign | out);
}

void orc_cast_f16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_fp16_to_float(src[i]);
}
void orc_cast_f32_to_f16_rne(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_float_to_fp16_rne(src[i]);
}
void orc_cast_f32_to_f16_ref_scalar(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_float_to_fp16_ref_scalar(src[i]);
}

/* ------------------------------------------------------------------------ */
/* Paged addressing: metal_runtime.mm:2266-2273, tests/test_paged_flash.cpp:36-45 */
/* ------------------------------------------------------------------------ */
static inline size_t kv_elem(const uint32_t* pt_flat, const uint32_t* pt_off, uint32_t req,
                             uint32_t pos, uint32_t kv_h, uint32_t P, uint32_t KVH, uint32_t D) {
    uint32_t page_idx = pos / P, slot = pos % P;
    uint32_t page_id = pt_flat[pt_off[req] + page_idx];
    return (size_t)page_id * ((size_t)P * KVH * D) + (size_t)slot * ((size_t)KVH * D) +
           (size_t)kv_h * D;
}

/*
 * Two-pass fp32 paged attention: tests/test_paged_flash.cpp:17-91
 * (cpuPagedFlashAttention), with the kernel's edge rules added:
 *   S == 0 -> zeros (metal_runtime.mm:2254-2257); every score masked -> zeros
 *   (inv_l guard, metal_runtime.mm:2333). GQA map kv_h = h*KVH/H (mm:2237);
 *   causal rule kv_pos > q_pos masked (mm:2286). `scale` replaces the
 *   reference's implicit 1/sqrt(D) (mm:7133); pass that value for parity.
 * q, out: fp32 [batch, H, D]; k_pages, v_pages: fp16 bits.
 */
void orc_paged_attention(const float* q, const uint16_t* k_pages, const uint16_t* v_pages,
                         const uint32_t* pt_flat, const uint32_t* pt_off,
                         const uint32_t* seq_lens, const uint32_t* q_pos, uint32_t batch,
                         uint32_t H, uint32_t KVH, uint32_t D, uint32_t P, int causal, float scale,
                         float* out) {
    for (uint32_t r = 0; r < batch; ++r) {
        uint32_t S = seq_lens[r];
        float* scores = (float*)malloc(sizeof(float) * (S ? S : 1));
        for (uint32_t h = 0; h < H; ++h) {
            uint32_t kv_h = (uint32_t)(((uint64_t)h * KVH) / H);
            const float* qrow = q + ((size_t)r * H + h) * D;
            float* orow = out + ((size_t)r * H + h) * D;
            float mx = -INFINITY;
            for (uint32_t pos = 0; pos < S; ++pos) {
                const uint16_t* krow = k_pages + kv_elem(pt_flat, pt_off, r, pos, kv_h, P, KVH, D);
                float dot = 0.0f;
                for (uint32_t d = 0; d < D; ++d) dot += qrow[d] * orc_fp16_to_float(krow[d]);
                float s = dot * scale;
                if (causal && pos > q_pos[r]) s = -INFINITY;
                scores[pos] = s;
                if (s > mx) mx = s;
            }
            float sum = 0.0f;
            for (uint32_t pos = 0; pos < S; ++pos) {
                float e = (scores[pos] == -INFINITY) ? 0.0f : expf(scores[pos] - mx);
                scores[pos] = e;
                sum += e;
            }
            float inv = (sum > 0.0f) ? 1.0f / sum : 0.0f;
            for (uint32_t d = 0; d < D; ++d) orow[d] = 0.0f;
            for (uint32_t pos = 0; pos < S; ++pos) {
                const uint16_t* vrow = v_pages + kv_elem(pt_flat, pt_off, r, pos, kv_h, P, KVH, D);
                float w = scores[pos];
                if (w == 0.0f) continue;
                for (uint32_t d = 0; d < D; ++d) orow[d] += w * orc_fp16_to_float(vrow[d]);
            }
            for (uint32_t d = 0; d < D; ++d) orow[d] *= inv;
        }
        free(scores);
    }
}

/*
 * The MSL kernel's tiled online-softmax recurrence, metal_runtime.mm:2216-2335:
 * per tile of `tile` tokens: scores, tile max, m_new = max(m, tile_max),
 * alpha = (m == -inf) ? 0 : exp(m - m_new), e_s = (score == -inf) ? 0 :
 * exp(score - m_new), o = o*alpha + sum_s e_s*V, l = l*alpha + sum_s e_s;
 * O = o * (l > 0 ? 1/l : 0). Optionally restricted to tokens [t0, t1) and
 * returning the un-normalised state (o, m, l) instead of O: that is the
 * split-KV partial whose combine is orc_lse_combine below.
 *   o_part: fp32 [batch, H, D] (un-normalised when ml_out != NULL)
 *   ml_out: fp32 [batch, H, 2] = (m, l), or NULL for the normalised output.
 */
void orc_paged_attention_tiled(const float* q, const uint16_t* k_pages, const uint16_t* v_pages,
                               const uint32_t* pt_flat, const uint32_t* pt_off,
                               const uint32_t* seq_lens, const uint32_t* q_pos, uint32_t batch,
                               uint32_t H, uint32_t KVH, uint32_t D, uint32_t P, int causal,
                               float scale, uint32_t tile, uint32_t t0, uint32_t t1, float* o_part,
                               float* ml_out) {
    float* sc = (float*)malloc(sizeof(float) * tile);
    float* acc = (float*)malloc(sizeof(float) * D);
    for (uint32_t r = 0; r < batch; ++r) {
        uint32_t S = seq_lens[r];
        uint32_t lo = t0 < S ? t0 : S, hi = t1 < S ? t1 : S;
        for (uint32_t h = 0; h < H; ++h) {
            uint32_t kv_h = (uint32_t)(((uint64_t)h * KVH) / H);
            const float* qrow = q + ((size_t)r * H + h) * D;
            float* orow = o_part + ((size_t)r * H + h) * D;
            float m = -INFINITY, l = 0.0f;
            for (uint32_t d = 0; d < D; ++d) orow[d] = 0.0f;
            for (uint32_t ts = lo; ts < hi; ts += tile) {
                uint32_t n = (hi - ts < tile) ? hi - ts : tile;
                float tmax = -INFINITY;
                for (uint32_t i = 0; i < n; ++i) {
                    uint32_t pos = ts + i;
                    const uint16_t* krow =
                        k_pages + kv_elem(pt_flat, pt_off, r, pos, kv_h, P, KVH, D);
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < D; ++d) dot += qrow[d] * orc_fp16_to_float(krow[d]);
                    float s = dot * scale;
                    if (causal && pos > q_pos[r]) s = -INFINITY;
                    sc[i] = s;
                    tmax = fmaxf(tmax, s);
                }
                float m_new = fmaxf(m, tmax);
                float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
                float tsum = 0.0f;
                for (uint32_t i = 0; i < n; ++i) {
                    float e = (sc[i] == -INFINITY) ? 0.0f : expf(sc[i] - m_new);
                    sc[i] = e;
                    tsum += e;
                }
                for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
                for (uint32_t i = 0; i < n; ++i) {
                    if (sc[i] == 0.0f) continue;
                    const uint16_t* vrow =
                        v_pages + kv_elem(pt_flat, pt_off, r, ts + i, kv_h, P, KVH, D);
                    for (uint32_t d = 0; d < D; ++d) acc[d] += sc[i] * orc_fp16_to_float(vrow[d]);
                }
                for (uint32_t d = 0; d < D; ++d) orow[d] = orow[d] * alpha + acc[d];
                l = l * alpha + tsum;
                m = m_new;
            }
            if (ml_out) {
                ml_out[((size_t)r * H + h) * 2 + 0] = m;
                ml_out[((size_t)r * H + h) * 2 + 1] = l;
            } else {
                float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
                for (uint32_t d = 0; d < D; ++d) orow[d] *= inv;
            }
        }
    }
    free(sc);
    free(acc);
}

/*
 * Log-sum-exp combine of `parts` split-KV partials (the step that follows the
 * gather of per-rank / per-CTA partials). The reference kernel has no split; the
 * rule is the one its per-tile update applies between tiles (mm:2304-2329),
 * applied between partials: m* = max_k m_k, w_k = (m_k == -inf) ? 0 :
 * exp(m_k - m*), l = sum_k l_k w_k, O = sum_k o_k w_k * (l > 0 ? 1/l : 0).
 *   o_parts: fp32 [parts, rows, D] un-normalised; ml_parts: fp32 [parts, rows, 2].
 */
void orc_lse_combine(const float* o_parts, const float* ml_parts, uint32_t parts, size_t rows,
                     uint32_t D, float* out) {
    for (size_t row = 0; row < rows; ++row) {
        float mstar = -INFINITY;
        for (uint32_t k = 0; k < parts; ++k)
            mstar = fmaxf(mstar, ml_parts[((size_t)k * rows + row) * 2]);
        float l = 0.0f;
        float* orow = out + row * D;
        for (uint32_t d = 0; d < D; ++d) orow[d] = 0.0f;
        for (uint32_t k = 0; k < parts; ++k) {
            float mk = ml_parts[((size_t)k * rows + row) * 2];
            float lk = ml_parts[((size_t)k * rows + row) * 2 + 1];
            float w = (mk == -INFINITY) ? 0.0f : expf(mk - mstar);
            l += lk * w;
            const float* ok = o_parts + ((size_t)k * rows + row) * D;
            for (uint32_t d = 0; d < D; ++d) orow[d] += ok[d] * w;
        }
        float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
        for (uint32_t d = 0; d < D; ++d) orow[d] *= inv;
    }
}

/*
 * Chunked (multi-token) causal paged attention. The reference has no paged
 * multi-token kernel; its CPU backend defines multi-token attention as a loop
 * of single-token causal steps at positions base+t
 * (compiler/runtime/operator_backend.cpp:906-968), each of which attends over
 * [0, base+t] (attention_cpu.cpp:437). Here all K/V rows are already in the
 * pool; query i of request r sits at position q_start[r] + i and sees
 * kv_pos <= q_start[r] + i, kv_pos < seq_lens[r].
 *   q, out: fp32 [sum_r q_len[r], H, D], requests concatenated in order.
 */
void orc_paged_prefill(const float* q, const uint16_t* k_pages, const uint16_t* v_pages,
                       const uint32_t* pt_flat, const uint32_t* pt_off, const uint32_t* seq_lens,
                       const uint32_t* q_start, const uint32_t* q_len, uint32_t batch, uint32_t H,
                       uint32_t KVH, uint32_t D, uint32_t P, float scale, float* out) {
    size_t row0 = 0;
    for (uint32_t r = 0; r < batch; ++r) {
        for (uint32_t i = 0; i < q_len[r]; ++i) {
            uint32_t qp = q_start[r] + i;
            uint32_t S = seq_lens[r];
            /* one single-token causal step for request r */
            uint32_t one_off[2] = {pt_off[r], pt_off[r + 1]};
            orc_paged_attention(q + (row0 + i) * H * D, k_pages, v_pages, pt_flat, one_off, &S, &qp,
                                1, H, KVH, D, P, 1, scale, out + (row0 + i) * H * D);
        }
        row0 += q_len[r];
    }
}

/* ------------------------------------------------------------------------ */
/* KV writers / readers                                                      */
/* ------------------------------------------------------------------------ */

/* scatter_kv_paged_batched_f16, metal_runtime.mm:405-424: one row per request.
 * src fp16 [batch, KVH, D]; dst index = page_ids[r]*E + slots[r]*KVH*D + kv*D + d. */
void orc_scatter_kv_paged_batched_f16(const uint16_t* src, uint16_t* page_storage,
                                      const uint32_t* page_ids, const uint32_t* slots,
                                      uint32_t P, uint32_t KVH, uint32_t D, uint32_t batch) {
    size_t E = (size_t)P * KVH * D, total = (size_t)batch * KVH * D;
    for (size_t gid = 0; gid < total; ++gid) {
        uint32_t dim = (uint32_t)(gid % D);
        size_t tmp = gid / D;
        uint32_t kv = (uint32_t)(tmp % KVH);
        size_t req = tmp / KVH;
        size_t dst = (size_t)page_ids[req] * E + (size_t)slots[req] * ((size_t)KVH * D) +
                     (size_t)kv * D + dim;
        page_storage[dst] = src[gid];
    }
}

/* scatter_kv_paged_f16/_f32, metal_runtime.mm:468-512: src [KVH, tokens, D];
 * absolute slot = start_slot + token walked through page_table. */
void orc_scatter_kv_paged(const void* src, void* page_storage, const uint32_t* page_table,
                          uint32_t P, uint32_t KVH, uint32_t D, uint32_t tokens,
                          uint32_t start_slot, uint32_t dtype_bytes) {
    size_t E = (size_t)P * KVH * D, total = (size_t)D * KVH * tokens;
    for (size_t gid = 0; gid < total; ++gid) {
        uint32_t dim = (uint32_t)(gid % D);
        size_t tmp = gid / D;
        uint32_t token = (uint32_t)(tmp % tokens);
        uint32_t kv = (uint32_t)(tmp / tokens);
        uint32_t abs_slot = start_slot + token;
        uint32_t page_idx = abs_slot / P, slot = abs_slot % P;
        size_t dst = (size_t)page_table[page_idx] * E + (size_t)slot * KVH * D + (size_t)kv * D + dim;
        memcpy((char*)page_storage + dst * dtype_bytes, (const char*)src + gid * dtype_bytes,
               dtype_bytes);
    }
}

/* gather_kv_pages_f16/_f32, metal_runtime.mm:328-370: dst [KVH, num_tokens, D]. */
void orc_gather_kv_pages(const void* page_storage, const uint32_t* page_table, void* dst,
                         uint32_t P, uint32_t KVH, uint32_t D, uint32_t num_tokens,
                         uint32_t dtype_bytes) {
    size_t E = (size_t)P * KVH * D, total = (size_t)KVH * num_tokens * D;
    for (size_t gid = 0; gid < total; ++gid) {
        uint32_t dim = (uint32_t)(gid % D);
        size_t tmp = gid / D;
        uint32_t tok = (uint32_t)(tmp % num_tokens);
        uint32_t head = (uint32_t)(tmp / num_tokens);
        uint32_t page_idx = tok / P, slot = tok % P;
        size_t so = (size_t)page_table[page_idx] * E + (size_t)slot * KVH * D + (size_t)head * D + dim;
        memcpy((char*)dst + gid * dtype_bytes, (const char*)page_storage + so * dtype_bytes,
               dtype_bytes);
    }
}

/* ------------------------------------------------------------------------ */
/* Page allocator: compiler/runtime/paged_kv.cpp:10-81                        */
/* ------------------------------------------------------------------------ */
typedef struct {
    uint32_t capacity;
    uint32_t* free_list; /* LIFO stack, id 0 on top of a fresh pool (paged_kv.cpp:10-17) */
    size_t n_free, in_use;
} orc_pool;

orc_pool* orc_pool_create(uint32_t capacity) {
    orc_pool* p = (orc_pool*)malloc(sizeof(orc_pool));
    p->capacity = capacity;
    p->free_list = (uint32_t*)malloc(sizeof(uint32_t) * (capacity ? capacity : 1));
    p->n_free = 0;
    for (uint32_t i = capacity; i-- > 0;) p->free_list[p->n_free++] = i;
    p->in_use = 0;
    return p;
}
void orc_pool_destroy(orc_pool* p) { free(p->free_list); free(p); }
/* paged_kv.cpp:19-25 */
int orc_pool_allocate(orc_pool* p, uint32_t* id) {
    if (p->n_free == 0) return 0;
    *id = p->free_list[--p->n_free];
    ++p->in_use;
    return 1;
}
/* paged_kv.cpp:37-42 */
void orc_pool_release(orc_pool* p, uint32_t id) { p->free_list[p->n_free++] = id; --p->in_use; }
size_t orc_pool_in_use(const orc_pool* p) { return p->in_use; }
size_t orc_pool_free(const orc_pool* p) { return p->n_free; }

/* RequestKVState::extend_one_token, paged_kv.cpp:53-66. State is (pages, n_pages,
 * tokens_in_last_page) owned by the caller; returns 0 on pool exhaustion. */
int orc_kvstate_extend(orc_pool* pool, uint32_t page_size, uint32_t* pages, size_t* n_pages,
                       uint32_t* tokens_in_last, uint32_t* page_id, uint32_t* slot) {
    if (page_size == 0) return 0;
    if (*n_pages == 0 || *tokens_in_last == page_size) {
        uint32_t id;
        if (!orc_pool_allocate(pool, &id)) return 0;
        pages[(*n_pages)++] = id;
        *tokens_in_last = 0;
    }
    *page_id = pages[*n_pages - 1];
    *slot = (*tokens_in_last)++;
    return 1;
}

/* ------------------------------------------------------------------------ */
/* QKV split + rotary embedding + cast (the step before the scatter)         */
/* ------------------------------------------------------------------------ */

/* computeRotaryCoefficients, compiler/runtime/quantization.cpp:795-823. */
void orc_compute_rotary(size_t position, size_t rotary_dim, float freq_base, float freq_scale,
                        float* cos_out, float* sin_out) {
    if (rotary_dim < 2) return;
    if (freq_base <= 0.0f) freq_base = 10000.0f;
    if (freq_scale == 0.0f) freq_scale = 1.0f;
    size_t pairs = rotary_dim / 2;
    float pos = (float)position;
    for (size_t i = 0; i < pairs; ++i) {
        float exponent = (float)(2 * i) / (float)rotary_dim;
        float inv_freq = powf(freq_base, -exponent);
        float angle = pos * inv_freq * freq_scale;
        cos_out[i] = cosf(angle);
        sin_out[i] = sinf(angle);
    }
}

/* batched_rope, metal_runtime.mm:287-314 (the CPU form is applyRotaryEmbedding,
 * quantization.cpp:773-793): adjacent pairs (2i, 2i+1) of every head, one cos/sin row per
 * request. data [batch, n_heads, head_dim], in place. */
void orc_batched_rope(float* data, const float* cos_t, const float* sin_t, uint32_t batch,
                      uint32_t n_heads, uint32_t head_dim, uint32_t rotary_dim) {
    uint32_t pairs = rotary_dim / 2;
    for (uint32_t r = 0; r < batch; ++r)
        for (uint32_t h = 0; h < n_heads; ++h)
            for (uint32_t i = 0; i < pairs; ++i) {
                float* d = data + ((size_t)r * n_heads + h) * head_dim;
                float c = cos_t[(size_t)r * pairs + i], s = sin_t[(size_t)r * pairs + i];
                volatile float a0 = d[2 * i] * c, a1 = d[2 * i + 1] * s; /* volatile: no contraction */
                volatile float b0 = d[2 * i] * s, b1 = d[2 * i + 1] * c;
                d[2 * i] = a0 - a1;
                d[2 * i + 1] = b0 + b1;
            }
}

/* encodeQkvSplitRopeCast, metal_runtime.mm:7915-8025: strided_copy_f32 x3 (mm:447-457),
 * batched_rope on Q and K, cast_f32_to_f16 on K and V (mm:459-466, round to nearest even). */
void orc_qkv_split_rope_cast(const float* qkv, float* q, float* k, float* v, uint16_t* k16,
                             uint16_t* v16, const float* cos_t, const float* sin_t, uint32_t batch,
                             uint32_t num_heads, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t qkv_rows, uint32_t q_rows, uint32_t k_rows, uint32_t v_rows,
                             uint32_t rotary_dim) {
    for (uint32_t r = 0; r < batch; ++r) {
        memcpy(q + (size_t)r * q_rows, qkv + (size_t)r * qkv_rows, (size_t)q_rows * 4);
        memcpy(k + (size_t)r * k_rows, qkv + (size_t)r * qkv_rows + q_rows, (size_t)k_rows * 4);
        memcpy(v + (size_t)r * v_rows, qkv + (size_t)r * qkv_rows + q_rows + k_rows, (size_t)v_rows * 4);
    }
    if (rotary_dim > 0) {
        orc_batched_rope(q, cos_t, sin_t, batch, num_heads, head_dim, rotary_dim);
        orc_batched_rope(k, cos_t, sin_t, batch, kv_heads, head_dim, rotary_dim);
    }
    orc_cast_f32_to_f16_rne(k, k16, (size_t)batch * k_rows);
    orc_cast_f32_to_f16_rne(v, v16, (size_t)batch * v_rows);
}
