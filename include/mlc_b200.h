/*
 * mlc_b200.h - C ABI of the B200-native paged-attention path.
 *
 * Drop-in boundary for MLcompiler's paged flash-attention decode kernel, its
 * paged KV writers/readers and the host objects that feed them. MLcompiler has
 * no FFI layer: the surface being replaced is the member-function set of the
 * singleton mlc::runtime::MetalExecutor (compiler/runtime/metal_runtime.hpp)
 * plus the paged-KV classes (compiler/runtime/paged_kv.hpp) and the scheduler
 * interface (compiler/runtime/scheduler.hpp, batched_executor.hpp). Each entry
 * point below names the declaration it stands in for.
 *
 * Conventions
 *   - Plain C: opaque handles, raw pointers, sizes. No C++/torch types.
 *   - "device pointer" = CUDA global memory of the context's GPU (from
 *     mlc_alloc, cudaMalloc, or a torch tensor's data_ptr()).
 *   - "host array" = ordinary host memory; it is copied during the call and
 *     never retained (same contract as the reference's std::vector arguments,
 *     metal_runtime.mm:7101-7107).
 *   - Every function returning int returns an mlc_status; MLC_OK == 0.
 *     The reference returns bool: ok <=> MLC_OK.
 *   - encode_* calls are asynchronous on the context's stream and require an
 *     open pass (mlc_pass_begin), like the reference's encode* members which
 *     need an open forward-pass command buffer (metal_runtime.mm:7090).
 *     run_* calls validate their arguments, launch and wait.
 *   - A context is single-threaded by contract (paged_kv.hpp:25-27).
 *   - There is no CPU fallback anywhere behind this header: without a CUDA
 *     device mlc_ctx_create fails with MLC_ERR_NO_DEVICE.
 */
#ifndef MLC_B200_H
#define MLC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mlc_status {
    MLC_OK = 0,
    MLC_ERR_INVALID_ARG = 1,   /* the cases for which the reference returns false */
    MLC_ERR_NO_OPEN_PASS = 2,  /* encode_* without mlc_pass_begin (mm:7090, 7178) */
    MLC_ERR_CUDA = 3,          /* a CUDA runtime/driver call failed; see mlc_last_error */
    MLC_ERR_BOUNDS = 4,        /* page id / slot / length check failed (added checks) */
    MLC_ERR_UNSUPPORTED = 5,   /* shape outside what the kernels cover (head_dim > 256) */
    MLC_ERR_NO_DEVICE = 6,
    MLC_ERR_OOM = 7,
    MLC_ERR_DEVICE_FLAG = 8    /* a kernel recorded an error word; see mlc_device_error_word */
} mlc_status;

typedef enum mlc_dtype { MLC_F32 = 0, MLC_F16 = 1 } mlc_dtype;

/* Bits of the device-written error word (never a trap, never a hang). */
#define MLC_DEVERR_WAIT_TIMEOUT 0x1u  /* a bounded mbarrier wait ran out */
#define MLC_DEVERR_BAD_PAGE 0x2u      /* page id >= capacity seen by a checking kernel */
#define MLC_DEVERR_BAD_SLOT 0x4u      /* slot >= page_size seen by a checking kernel */
#define MLC_DEVERR_BAD_TOKEN 0x8u     /* token id >= vocabulary size seen by the embedding kernel */

typedef struct mlc_ctx mlc_ctx;

/* ---- context: replaces MetalExecutor::Instance() (metal_runtime.mm:5774) ------
 * One context per GPU. `stream` is a cudaStream_t to enqueue on, or NULL to let
 * the context create its own non-blocking stream. */
int mlc_ctx_create(int device, void* stream, mlc_ctx** out);
void mlc_ctx_destroy(mlc_ctx* ctx);
/* isAvailable() (metal_runtime.hpp:26): 1 when the context owns a usable device. */
int mlc_ctx_available(const mlc_ctx* ctx);
/* Text of the most recent failure on this context (valid until the next call). */
const char* mlc_last_error(const mlc_ctx* ctx);
/* Reads and clears the device error word (synchronises the stream first). */
int mlc_device_error_word(mlc_ctx* ctx, uint32_t* word);
/* The stream the context enqueues on (cudaStream_t). */
void* mlc_ctx_stream(const mlc_ctx* ctx);
/* Number of kernels this context has launched since creation. */
uint64_t mlc_ctx_launch_count(const mlc_ctx* ctx);
/* Number of device-memory and pinned-host allocations this context has made since
 * creation (mlc_alloc, plan buffers, staging chunks, the split-KV workspace, exchange
 * buffers). A caller that must stay allocation-free in steady state can assert that the
 * count stops moving. */
uint64_t mlc_ctx_alloc_count(const mlc_ctx* ctx);
/* Limit, in polls (about a microsecond each), of the waits on flags that another GPU writes
 * (the peer exchange kernel). 0 restores the default of about a second. When a wait runs
 * out, the kernel records MLC_DEVERR_WAIT_TIMEOUT in the device error word, writes no
 * output and returns; the context stays usable. */
int mlc_ctx_set_wait_limit(mlc_ctx* ctx, uint32_t polls);
/* Profiling aid (the reference's are env-gated wall-clock tables,
 * compiler/runtime/batched_walker.cpp:100-125): with MLC_B200_TRACE=1 in the
 * environment when the context is created, every warp of the decode attention
 * kernel records 8 %globaltimer stamps (entry, copies issued, first tile landed,
 * first piece computed, partial published / merged, merge done, merge started, exit).
 * Copies the stamps of the most recent launch (previous = 0) or of the one before it
 * (previous = 1) as [rows][4][8] u64 nanoseconds, a row being 4 consecutive warps (one
 * row per CTA, two for the 8-warp CTAs of unit mode); returns the number of rows. */
uint32_t mlc_ctx_read_trace(mlc_ctx* ctx, unsigned long long* out, size_t max_words, int previous);

/* ---- buffers: allocateScratchBuffer / releaseScratchBuffer / uploadToBuffer /
 * downloadFromBuffer (metal_runtime.hpp:693-696) and getOrAllocCachedBuffer
 * (metal_runtime.hpp:703). upload/download are synchronous. */
void* mlc_alloc(mlc_ctx* ctx, size_t bytes);
void mlc_free(mlc_ctx* ctx, void* buffer);
int mlc_upload(mlc_ctx* ctx, void* buffer, const void* src, size_t bytes, size_t dst_offset);
int mlc_download(mlc_ctx* ctx, const void* buffer, void* dst, size_t bytes, size_t src_offset);
void* mlc_cached_buffer(mlc_ctx* ctx, const char* name, size_t bytes);
/* Size of the mlc_alloc / mlc_cached_buffer allocation that starts at `buffer`,
 * or 0 if the pointer is not one of the context's own. */
size_t mlc_buffer_bytes(const mlc_ctx* ctx, const void* buffer);

/* ---- pass bracketing: beginForwardPassCB / hasForwardPassCB / flushForwardPassCB
 * (metal_runtime.hpp:181-183). flush waits for the stream and reports
 * MLC_ERR_DEVICE_FLAG if a kernel of the pass recorded an error word. */
int mlc_pass_begin(mlc_ctx* ctx);
int mlc_pass_is_open(const mlc_ctx* ctx);
int mlc_pass_flush(mlc_ctx* ctx);

/* ---- KV writers / readers ------------------------------------------------------
 * Page layout everywhere: [page_size_tokens, n_kv_heads, head_dim] token-major,
 * page i at element offset i * page_size_tokens * n_kv_heads * head_dim
 * (paged_kv.hpp:101-105).
 *
 * capacity_pages: number of pages `page_storage` holds, used for the added
 * bounds checks; pass 0 when unknown (then, like the reference, ids are not
 * checked - except that buffers obtained from mlc_alloc are still checked
 * against their recorded size). */

/* scatterKVPagedBatched (metal_runtime.hpp:680-687; kernel
 * scatter_kv_paged_batched_f16, metal_runtime.mm:405-424): one new fp16 row per
 * request. src: device fp16 [batch, n_kv_heads, head_dim]; page_ids / slots_in_page:
 * host u32 [batch]. Synchronous. */
int mlc_run_scatter_kv_paged_batched_f16(mlc_ctx* ctx, void* page_storage,
                                         const uint32_t* page_ids, const uint32_t* slots_in_page,
                                         size_t page_size_tokens, size_t n_kv_heads,
                                         size_t head_dim, size_t batch, const void* src,
                                         size_t capacity_pages);
/* encodeScatterKVPagedBatched (metal_runtime.hpp:526-533). Asynchronous. */
int mlc_encode_scatter_kv_paged_batched_f16(mlc_ctx* ctx, void* page_storage,
                                            const uint32_t* page_ids,
                                            const uint32_t* slots_in_page,
                                            size_t page_size_tokens, size_t n_kv_heads,
                                            size_t head_dim, size_t batch, const void* src,
                                            size_t capacity_pages);
/* K and V rows of one layer in ONE launch (the reference issues two dispatches,
 * batched_walker.cpp:304-309). Asynchronous. */
int mlc_encode_scatter_kv_pair_paged_batched_f16(mlc_ctx* ctx, void* k_page_storage,
                                                 void* v_page_storage, const uint32_t* page_ids,
                                                 const uint32_t* slots_in_page,
                                                 size_t page_size_tokens, size_t n_kv_heads,
                                                 size_t head_dim, size_t batch, const void* k_src,
                                                 const void* v_src, size_t capacity_pages);
/* scatterKVPaged (metal_runtime.hpp:666-674; kernels scatter_kv_paged_f16/_f32,
 * metal_runtime.mm:468-512): multi-token scatter of one request. src: device
 * [n_kv_heads, tokens, head_dim]; page_table: host u32 [n_page_table]. Synchronous. */
int mlc_run_scatter_kv_paged(mlc_ctx* ctx, void* page_storage, const uint32_t* page_table,
                             size_t n_page_table, size_t page_size_tokens, size_t n_kv_heads,
                             size_t head_dim, size_t tokens, size_t start_slot, const void* src,
                             size_t dtype_bytes, size_t capacity_pages);
/* gatherKVPages (metal_runtime.hpp:619-626; kernels gather_kv_pages_f16/_f32,
 * metal_runtime.mm:328-370): paged -> contiguous [n_kv_heads, num_tokens, head_dim]. */
int mlc_run_gather_kv_pages(mlc_ctx* ctx, const void* page_storage, const uint32_t* page_table,
                            size_t n_page_table, size_t page_size_tokens, size_t n_kv_heads,
                            size_t head_dim, size_t num_tokens, void* dst, size_t dtype_bytes,
                            size_t capacity_pages);

/* ---- paged flash-attention decode ------------------------------------------------
 * O[r,h,:] = softmax_s(scale * Q[r,h,:].K[r,s,kv_h,:] + mask) . V[r,s,kv_h,:],
 * s in [0, seq_lens[r]), kv_h = h * kv_heads / num_heads, mask = -inf where
 * apply_causal and s > q_positions[r]; seq_lens[r] == 0 or a fully masked row
 * gives zeros (kernel paged_flash_attention, metal_runtime.mm:2216-2335).
 *
 *   q, o            device [batch, num_heads, head_dim], fp32 (the reference's
 *                   type, metal_runtime.hpp:632-636) or fp16, per q_dtype / o_dtype
 *   k_pages,v_pages device fp16 paged pools
 *   page_tables_flat, page_table_offsets[batch+1], seq_lens[batch],
 *   q_positions[batch]   host u32 arrays
 *   scale           multiplies the scores; the reference hard-codes
 *                   1/sqrt(head_dim) (metal_runtime.mm:7133) - pass a value <= 0
 *                   to get exactly that.
 */
/* runPagedFlashAttention (metal_runtime.hpp:645-658). Validates as
 * metal_runtime.mm:7742-7750, launches, waits. */
int mlc_run_paged_flash_attention(mlc_ctx* ctx, const void* q, const void* k_pages,
                                  const void* v_pages, void* o,
                                  const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                  const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                  const uint32_t* q_positions, size_t batch, size_t num_heads,
                                  size_t kv_heads, size_t head_dim, size_t page_size_tokens,
                                  int apply_causal, float scale, int q_dtype, int o_dtype,
                                  size_t capacity_pages);
/* encodePagedFlashAttention (metal_runtime.hpp:510-523). Asynchronous. */
int mlc_encode_paged_flash_attention(mlc_ctx* ctx, const void* q, const void* k_pages,
                                     const void* v_pages, void* o,
                                     const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                     const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                     const uint32_t* q_positions, size_t batch, size_t num_heads,
                                     size_t kv_heads, size_t head_dim, size_t page_size_tokens,
                                     int apply_causal, float scale, int q_dtype, int o_dtype,
                                     size_t capacity_pages);

/* Selects the kernel family used by the attention entry points of this context:
 * 0 = automatic (TMA + tensor-core split-KV kernel when the shape allows it,
 * otherwise the general kernel), 1 = always the general kernel. Both are CUDA. */
int mlc_ctx_set_attention_kernel(mlc_ctx* ctx, int which);
/* Which family the most recent attention call used: 0 none yet, 1 general, 2 TMA decode,
 * 3 tcgen05 chunked prefill. */
int mlc_ctx_last_attention_kernel(const mlc_ctx* ctx);

/* ---- device-resident plans --------------------------------------------------------
 * The reference rebuilds and re-uploads page_tables_flat / offsets / seq_lens /
 * q_positions for every layer of a pass although they are identical across layers
 * (compiler/runtime/batched_walker.cpp:316-325, metal_runtime.mm:7092-7107). A plan
 * holds one pass's tables - and, optionally, the (page, slot) each request's new
 * K/V row goes to (batched_walker.cpp:127-142) - on the device, so the per-layer
 * calls carry no host arrays. The host-array entry points above build and cache
 * such plans internally. */
typedef struct mlc_attn_plan mlc_attn_plan;
int mlc_attn_plan_create(mlc_ctx* ctx, const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                         const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                         const uint32_t* q_positions, const uint32_t* page_ids /* may be NULL */,
                         const uint32_t* slots_in_page /* may be NULL */, size_t batch,
                         size_t num_heads, size_t kv_heads, size_t head_dim,
                         size_t page_size_tokens, int apply_causal, size_t capacity_pages,
                         mlc_attn_plan** out);
void mlc_attn_plan_destroy(mlc_ctx* ctx, mlc_attn_plan* plan);
/* The next decode step's tables into the same plan (same head shape, page size, causal flag and
 * capacity; batch may change): what the walker's per-step table rebuild
 * (batched_walker.cpp:127-149, 316-325) becomes. Reuses the plan's pinned and device buffers; the
 * upload is ordered on the context's stream behind the kernels already enqueued with the old
 * tables. Not inside a graph capture. */
int mlc_attn_plan_update(mlc_ctx* ctx, mlc_attn_plan* plan, const uint32_t* page_tables_flat,
                         size_t n_page_tables_flat, const uint32_t* page_table_offsets,
                         const uint32_t* seq_lens, const uint32_t* q_positions, const uint32_t* page_ids,
                         const uint32_t* slots_in_page, size_t batch);
/* encodePagedFlashAttention (metal_runtime.hpp:510-523) with the tables taken from `plan`. */
int mlc_encode_paged_flash_attention_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                             const void* k_pages, const void* v_pages, void* o,
                                             float scale, int q_dtype, int o_dtype);
/* The two encodeScatterKVPagedBatched calls of a layer (batched_walker.cpp:304-309) as
 * one launch, page ids and slots taken from `plan`. */
int mlc_encode_scatter_kv_pair_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, void* k_page_storage,
                                       void* v_page_storage, const void* k_src, const void* v_src);

/* One layer of a decode step in ONE launch: what the reference's walker issues as two
 * encodeScatterKVPagedBatched calls followed by encodePagedFlashAttention
 * (batched_walker.cpp:299-331). The attention kernel writes each request's new K/V
 * row (k_new / v_new: device fp16 [batch, kv_heads, head_dim]) to the (page, slot) the
 * plan was created with and attends over the pool including that row. Requirements
 * for the single-launch form (otherwise the call transparently issues the scatter
 * and the attention as two launches): the plan was created with page_ids /
 * slots_in_page pointing at token seq_lens[r]-1 of every request and q_positions[r]
 * == seq_lens[r]-1, as in a decode step.
 * Stream-order contract of the single-launch form: the kernel is launched with
 * programmatic stream serialisation and starts fetching K/V pages while earlier work
 * on the stream is still finishing; Q, k_new and v_new are read only after that work
 * has completed. Therefore pool rows OTHER than this step's new rows must not be
 * written by OTHER parties' work that is still in flight on the stream when this call
 * is enqueued (they were written by earlier steps; a pass_flush / stream sync between
 * steps, or any ordinary kernel launch in between, satisfies this). The library's own
 * step launches need no such care: a launch whose pools were written by one of the two
 * decode launches enqueued just before it on this context (passes of one or two
 * layers) does not fetch anything before the earlier work has completed. */
int mlc_encode_paged_decode_step_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                         const void* k_new, const void* v_new, void* k_pages,
                                         void* v_pages, void* o, float scale, int q_dtype, int o_dtype);

/* Planned attention that allocates nothing (no counterpart in the reference, whose
 * kernel never splits a sequence and so needs no scratch). For callers that must not
 * allocate device memory when they call: a server that has given the whole GPU to its
 * own memory pool (a later cudaMalloc would fail or fragment it), or a decode loop that
 * cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply. Same
 * arguments and result as mlc_encode_paged_flash_attention_planned, but the split-KV
 * scratch is a fixed 8 MiB array inside the library (mlc_static_scratch_bytes(); every
 * GPU that loads the library holds it until exit) instead of the context's growing
 * workspace; the call makes no cudaMalloc / cudaFree and no host allocation.
 *   - Limit: the array is used as two halves of 4 MiB, each ending with a 16 KiB block of
 *     arrival counters. A batch whose split or cut requests need more than 4 MiB - 16 KiB
 *     of partials (about 450 request pieces at head_dim 64), or that cuts more than 4096
 *     (request, head) units over CTAs, is rejected with MLC_ERR_UNSUPPORTED and a message
 *     naming the sizes; use the regular entry point for it. The plan itself is created
 *     beforehand with mlc_attn_plan_create, which does allocate.
 *   - The first call on a device resolves the array's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture.
 *   - All calls on a GPU share the array and it keeps the last call's contents. The
 *     partials need no initial value (each is fully written before it is read). The
 *     counter blocks do: they rely on the array's zero initialisation at library load,
 *     every launch leaves them at zero again, they sit at a fixed place that no plan's
 *     partials can reach, and the context re-zeroes them after a kernel reported a
 *     device error. Two such calls that overlap on the GPU - different contexts or
 *     streams of the same device - race on the array. Consecutive calls on one context
 *     are safe: they are stream-ordered and alternate between the two halves (counted
 *     per context over calls of this entry point only). */
size_t mlc_static_scratch_bytes(void);
int mlc_encode_paged_flash_attention_planned_static(mlc_ctx* ctx, const mlc_attn_plan* plan,
                                                    const void* q, const void* k_pages,
                                                    const void* v_pages, void* o, float scale,
                                                    int q_dtype, int o_dtype);

/* ---- split-KV across GPUs (no counterpart in the reference: it has one device) -------
 * A rank that holds only a slice of every request's pages computes, over its
 * slice, the un-normalised state of the online softmax instead of O:
 *   o_partial  fp32 [batch, num_heads, head_dim] = sum_s exp(score_s - m) V_s
 *   ml_partial fp32 [batch, num_heads, 2]        = (m, l), m in natural-log units
 * After the ranks' partials have been gathered (NCCL), mlc_encode_lse_combine
 * merges `parts` of them laid out [parts, rows, head_dim] / [parts, rows, 2]:
 *   m* = max_k m_k, w_k = exp(m_k - m*), O = sum_k o_k w_k / sum_k l_k w_k
 * - between partials, the rule the reference kernel applies between tiles
 * (metal_runtime.mm:2304-2329). */
int mlc_encode_paged_attention_partial_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                               const void* k_pages, const void* v_pages,
                                               float* o_partial, float* ml_partial, float scale,
                                               int q_dtype);
int mlc_encode_lse_combine(mlc_ctx* ctx, const float* o_parts, const float* ml_parts, size_t parts,
                           size_t rows, size_t head_dim, void* out, int o_dtype);

/* All layers of one decode pass in one call - the layer loop of the reference's walker
 * (batched_walker.cpp:299-331) on this side of the boundary: the result is that of, for l in
 * [0, n_layers), mlc_encode_paged_decode_step_planned(plan, q[l], k_new[l], v_new[l], k_pages[l],
 * v_pages[l], o[l]). The arrays are host arrays of device pointers, read during the call.
 * CONTRACT: every layer's q / k_new / v_new must be complete when the work enqueued before this
 * call on the stream has finished - no layer's input may depend on another layer's output of the
 * same call (layers of a model whose attention inputs are produced ahead of time, or independent
 * layer pools as in a bandwidth benchmark; a transformer that feeds layer l's output into layer
 * l + 1 calls the per-layer entry point instead). Under that contract the library is free to
 * interleave the layers: when the plan keeps every (request, head) inside one CTA and was
 * created with page_ids / slots_in_page, the whole pass is ONE launch of at most 64 layers whose
 * (layer, request, head) work items are dealt to the SMs across layers, so that every SM gets
 * the same number of KV bytes whatever the spread of context lengths inside a layer and there
 * is no per-layer tail or launch hand-over; otherwise (or with MLC_B200_DECODE_PASS=0 in the
 * environment) it is one launch per layer. The pools of different layers must not overlap.
 * Stops at the first layer that fails and returns its status. */
int mlc_encode_paged_decode_pass_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, size_t n_layers,
                                         const void* const* q, const void* const* k_new,
                                         const void* const* v_new, void* const* k_pages,
                                         void* const* v_pages, void* const* o, float scale, int q_dtype,
                                         int o_dtype);

/* The same pass for a caller whose activations live in host memory (the reference's walker hands the
 * runtime host vectors per layer, batched_walker.cpp:299-331, and reads the result back): copies in,
 * kernels and copies out are pipelined over the layers inside the call.
 *   host_in  [n_layers] rows of [ Q: batch*H*D of q_dtype | new K: batch*KVH*D fp16 | new V: same ],
 *            pinned memory if the copies are to overlap the kernels
 *   dev_in   device staging buffer of the same size, caller-owned
 *   dev_o / host_o  [n_layers][batch][H][D] of o_dtype on the device and in host memory
 * The layers go in n_groups groups (0 = 5): group g's rows are copied on a copy stream while group
 * g-1 computes, its O rows go back on another stream while group g+1 computes. mlc_pass_flush waits
 * for the last copy back as well as for the context's stream: host_o is complete when it returns (the
 * stream itself is not held up by that copy, so an upload queued next - mlc_attn_plan_update for the
 * following step - runs beside it; a second host-buffer pass without a flush in between is ordered
 * behind the first one's copies).
 * Not capturable (MLC_ERR_UNSUPPORTED between mlc_graph_begin_capture and _end_capture). The streams
 * and events are created on the first call.
 * Zero-copy form: when the pass can run as one launch (see mlc_encode_paged_decode_pass_planned; the
 * same contract on the layers' independence holds) and host_in / host_o are pinned host memory that
 * the GPU can address (cudaHostAlloc, cudaHostRegister, torch pin_memory), there are no copies at
 * all: the kernel reads every Q / new K / new V row from host memory itself - once, one work item
 * ahead of its use - and stores O straight into host_o, so the transfers run beside the KV stream.
 * dev_in and dev_o are then left untouched (their contents after the call are unspecified either
 * way). host_o is complete when mlc_pass_flush returns. MLC_B200_DECODE_ZERO_COPY=0 in the
 * environment keeps the copy pipeline. */
int mlc_encode_paged_decode_pass_host(mlc_ctx* ctx, const mlc_attn_plan* plan, size_t n_layers,
                                      const void* host_in, void* dev_in, void* const* k_pages,
                                      void* const* v_pages, void* dev_o, void* host_o, float scale,
                                      int q_dtype, int o_dtype, size_t n_groups);

/* ---- QKV split + rotary embedding + cast, the step that feeds the scatter -------------
 * encodeQkvSplitRopeCast (metal_runtime.hpp:540-547; metal_runtime.mm:7915-8025: 3 x
 * strided_copy_f32 + 2 x batched_rope + 2 x cast_f32_to_f16 in one encoder) as ONE launch.
 *   qkv        device fp32 [batch, qkv_rows], row = [q_rows | k_rows | v_rows | ...]
 *   q, k, v    device fp32 [batch, q_rows / k_rows / v_rows]  (Q and K rotated)
 *   k_f16, v_f16 device fp16 copies of k, v (round to nearest even, like MSL half())
 *   cos_table, sin_table device fp32 [batch, rotary_dim / 2], one row per request
 *              (computeRotaryCoefficients, quantization.cpp:795-823; mlc_compute_rotary_coefficients)
 * Rotation of adjacent pairs (2i, 2i+1), i < rotary_dim / 2, of every head:
 *   y0 = x0*c - x1*s, y1 = x0*s + x1*c in fp32 without contraction (bit-exact against the CPU
 *   restatement). rotary_dim = 0 applies no rotation. Needs an open pass. */
int mlc_encode_qkv_split_rope_cast(mlc_ctx* ctx, const void* qkv, void* q, void* k, void* v, void* k_f16,
                                   void* v_f16, const void* cos_table, const void* sin_table, size_t batch,
                                   size_t num_heads, size_t kv_heads, size_t head_dim, size_t qkv_rows,
                                   size_t q_rows, size_t k_rows, size_t v_rows, size_t rotary_dim);
/* The same step fused with the two scatters that follow it in the walker
 * (batched_walker.cpp:299-309): the rotated K row and the V row of request r are written as
 * fp16 straight to (page_ids[r], slots_in_page[r]) of the pools held by `plan`, and Q is
 * written as q_dtype (fp32 like the reference, or fp16 for the attention kernel). Replaces 9
 * dispatches of the reference; no fp32 K/V and no fp16 staging buffers. Capturable. */
int mlc_encode_qkv_split_rope_scatter_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* qkv,
                                              void* q_out, int q_dtype, void* k_page_storage,
                                              void* v_page_storage, const void* cos_table,
                                              const void* sin_table, size_t qkv_rows, size_t rotary_dim);
/* The fused Q | K | V projection and the step above in one launch: weights = (num_heads + 2 kv_heads) *
 * head_dim rows of `cols` (quant, in, in_stride, input_kind, row_stride as in mlc_encode_matmul_quant_fused,
 * input_kind 0 or 2); the kernel that has added up four adjacent rows of a request rotates them, rounds
 * them to fp16 and writes Q to q_out [batch, num_heads * head_dim] (fp16) and K / V into the plan's
 * (page, slot) of the request - bit for bit what mlc_encode_matmul_quant_fused followed by
 * mlc_encode_qkv_split_rope_scatter_planned leaves there, without the fp32 [batch, qkv_rows] round trip and
 * its launch. head_dim must be a multiple of 4, q_out 16-byte aligned. */
int mlc_encode_matmul_qkv_rope_scatter_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, int quant, const void* weights,
                                               const void* in, size_t in_stride, int input_kind, size_t cols,
                                               size_t row_stride, void* q_out, void* k_page_storage,
                                               void* v_page_storage, const void* cos_table, const void* sin_table,
                                               size_t rotary_dim);
/* computeRotaryCoefficients (quantization.cpp:795-823) on the host: cos/sin of
 * position * freq_base^(-2i/rotary_dim) * freq_scale for i < rotary_dim / 2
 * (freq_base <= 0 -> 10000, freq_scale == 0 -> 1, as in the reference). */
int mlc_compute_rotary_coefficients(size_t position, size_t rotary_dim, float freq_base, float freq_scale,
                                    float* cos_out, float* sin_out);

/* ---- the other ops of the walker's decode step ------------------------------------------
 * What compiler/runtime/batched_walker.cpp:248-297 and :333-458 encode around attention, on
 * device buffers, onto the open pass (MLC_ERR_NO_OPEN_PASS otherwise, as every encode* of the
 * reference returns false without an open command buffer). Weights are device pointers: the
 * reference keeps them in a name-keyed buffer cache filled on first use, which a caller gets
 * from mlc_cached_buffer + mlc_upload. Activations are fp32 like the reference's. */

/* encodeRmsNormBatched (metal_runtime.hpp:474-479; kernel rms_norm_batched, metal_runtime.mm:166-209):
 * out[r, i] = in[r, i] * (1 / sqrt(mean(in[r, :]^2) + epsilon)) * weight[i], fp32, factors in the
 * order of operator_backend.cpp:186-204. weight: device fp32 [length]. out_f16 (may be NULL; no
 * counterpart in the reference) receives the same rows rounded to fp16. */
int mlc_encode_rms_norm_batched(mlc_ctx* ctx, const void* in, const void* weight, float epsilon, size_t batch,
                                size_t length, void* out, void* out_f16);
/* encodeAddBatched (metal_runtime.hpp:501-502; add_vectors, metal_runtime.mm:44-52): out = a + b. */
int mlc_encode_add_batched(mlc_ctx* ctx, const void* a, const void* b, void* out, size_t total_elements);
/* encodeSiluMulBatched (metal_runtime.hpp:505-506; feedforward_silu_mul, metal_runtime.mm:32-42):
 * out = gate / (1 + exp(-gate)) * up. */
int mlc_encode_silu_mul_batched(mlc_ctx* ctx, const void* gate, const void* up, void* out, size_t total_elements);
/* encodeGateUpSplitSiluMul (metal_runtime.hpp:549-552; metal_runtime.mm:8030-8088: two strided
 * copies + SiLU * mul in one encoder) as one launch. gate_up [batch, ffn_gate_up_rows] holds gate in
 * columns [0, ffn_inner) and up in [ffn_inner, 2 * ffn_inner); gate / up ([batch, ffn_inner]) receive
 * the copies and may be NULL; out [batch, ffn_inner]. */
int mlc_encode_gate_up_split_silu_mul(mlc_ctx* ctx, const void* gate_up, void* gate, void* up, void* out, size_t batch,
                                      size_t ffn_inner, size_t ffn_gate_up_rows);
/* encodeMatMulQ4_0Batched / encodeMatMulQ6KBatched (metal_runtime.hpp:481-498; kernels
 * q4_0_matmul_v3_batched, metal_runtime.mm:710-785, and q6_k_matmul_v3_batched, mm:1581-1655):
 * out[n, r] = sum_c W[r, c] * in[n, c]. weights: device bytes, `rows` rows of `row_stride` bytes in
 * the block format of quantization.cpp:71-74 (Q4_0: fp16 scale + 16 bytes per 32 weights) or
 * :142-147 (Q6_K: 210 bytes per 256 weights); in [batch, cols], out [batch, rows] fp32.
 * Tensor-core kernel: block integers exact, activations rounded to fp16, fp32 sums and scales.
 * Limits (MLC_ERR_UNSUPPORTED): batch <= 64, cols a whole number of blocks. Rows are copied
 * with 16-byte loads when weights and row_stride are 16-byte aligned (every real model's are:
 * cols a multiple of 256), with 2-byte loads otherwise. out and residual must be 16-byte aligned
 * when rows is a multiple of 4. */
int mlc_encode_matmul_q4_0_batched(mlc_ctx* ctx, const void* weights, const void* in, size_t batch, size_t rows,
                                   size_t cols, size_t row_stride, void* out);
int mlc_encode_matmul_q6k_batched(mlc_ctx* ctx, const void* weights, const void* in, size_t batch, size_t rows,
                                  size_t cols, size_t row_stride, void* out);
/* Embedding rows of a Q4_0 token table, dequantised on the device: the host loop of
 * batched_walker.cpp:183-208 (dequantizeRowTo per request, then one upload) as one launch, bit for
 * bit the CPU's rows. table: device bytes, `vocab` rows of row_stride bytes; token_ids: device
 * uint32 [batch]; out fp32 [batch, cols]. A token id >= vocab yields a zero row and
 * MLC_DEVERR_BAD_TOKEN in the device error word. */
int mlc_encode_embedding_q4_0(mlc_ctx* ctx, const void* table, size_t row_stride, const void* token_ids, size_t batch,
                              size_t cols, size_t vocab, void* out);
/* Greedy sampling on the device (no counterpart in the reference, whose scheduler takes the argmax of the
 * logits on the host, scheduler.cpp:101-118): out_ids[n] (uint32) = index of the first maximum of request n's
 * vocab logits. group_rows = 0 or >= vocab: logits is a plain [batch, vocab] array; otherwise the walker's
 * layout, groups of group_rows vocabulary rows, each group a [batch, rows of the group] array. */
int mlc_encode_argmax_rows(mlc_ctx* ctx, const void* logits, size_t batch, size_t vocab, size_t group_rows, void* out_ids);
/* The same mat-vec with its neighbours in the walker fused in (no counterpart in the reference).
 * input_kind 0: in = fp32 [batch, in_stride], as above.
 * input_kind 1: the input row n is SiLU(in[n, c]) * in[n, cols + c], computed on load (in = the
 *   gate | up buffer, in_stride >= 2 * cols: the step of batched_walker.cpp:379-394 without the
 *   intermediate buffers).
 * input_kind 2: in holds the activations in the kernel's operand format, written by
 *   mlc_encode_rms_norm_batched_packed (same size and shape as the fp32 buffer) - the kernel then
 *   skips its own conversion.
 * residual != NULL: out = residual + W in (the add of batched_walker.cpp:349 / :403).
 * quant: 0 = Q4_0, 1 = Q6_K. in_stride = 4-byte words between input rows. */
int mlc_encode_matmul_quant_fused(mlc_ctx* ctx, int quant, const void* weights, const void* in, size_t in_stride,
                                  int input_kind, const void* residual, size_t batch, size_t rows, size_t cols,
                                  size_t row_stride, void* out);
/* The gate | up projection with SiLU(gate) * up in its epilogue (batched_walker.cpp:364-394 in one launch):
 * weights = 2 * ffn_inner rows, the gate rows first, then the up rows (the layout of the walker's fused
 * ffn_gate_up tensor). Every row tile holds gate rows and the up rows that go with them, so the kernel that
 * has added up a gate sum also holds its up sum; packed [batch, ffn_inner] receives SiLU(gate) * up in the
 * operand format (input_kind 2 of the next mat-vec, the down projection). input_kind 0 or 2 as above.
 * ffn_inner must be divisible by 4. */
int mlc_encode_matmul_gate_up_silu_packed(mlc_ctx* ctx, int quant, const void* weights, const void* in, size_t in_stride,
                                          int input_kind, size_t batch, size_t ffn_inner, size_t cols, size_t row_stride,
                                          void* packed);
/* RMSNorm whose output goes to `packed` in the mat-vec kernel's operand format: per pair of columns
 * the 32-bit words {fp16(y0), fp16(y1)} and {fp16(y0 - hi0), fp16(y1 - hi1)} - 22 bits of every value,
 * in a buffer of the fp32 output's size. out (fp32) may be NULL. length must be divisible by 4. */
int mlc_encode_rms_norm_batched_packed(mlc_ctx* ctx, const void* in, const void* weight, float epsilon, size_t batch,
                                       size_t length, void* out, void* packed);

/* ---- chunked (multi-token) causal paged attention ------------------------------------
 * The reference runs a paged prefill as q_len single-token decode passes
 * (compiler/runtime/batched_executor.cpp:450-467); these entry points compute the same
 * result for all query tokens of all requests in one launch. Query i of request r sits
 * at position q_start[r] + i and attends to kv_pos <= q_start[r] + i (the mask rule of
 * metal_runtime.mm:2286, what compiler/runtime/operator_backend.cpp:906-968 computes for
 * seq_len > 1). Requires q_start[r] + q_len[r] <= seq_lens[r]: the chunk's K/V rows are
 * scattered into the pages first, the reference's order (batched_walker.cpp:299-331).
 *   q, o   [sum_r q_len[r], num_heads, head_dim], request after request
 *   tables as in mlc_encode_paged_flash_attention
 * With fp16 q and o, head_dim 128 and 64-token pages the work runs on tcgen05 tensor
 * cores (accumulators in tensor memory, operands staged by TMA); every other shape /
 * dtype runs the any-shape kernel, one row per query token.
 * mlc_ctx_last_attention_kernel reports 3 for the tcgen05 kernel. */
int mlc_run_paged_prefill_attention(mlc_ctx* ctx, const void* q, const void* k_pages, const void* v_pages,
                                    void* o, const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                    const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                    const uint32_t* q_start, const uint32_t* q_len, size_t batch,
                                    size_t num_heads, size_t kv_heads, size_t head_dim,
                                    size_t page_size_tokens, float scale, int q_dtype, int o_dtype,
                                    size_t capacity_pages);
int mlc_encode_paged_prefill_attention(mlc_ctx* ctx, const void* q, const void* k_pages, const void* v_pages,
                                       void* o, const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                       const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                       const uint32_t* q_start, const uint32_t* q_len, size_t batch,
                                       size_t num_heads, size_t kv_heads, size_t head_dim,
                                       size_t page_size_tokens, float scale, int q_dtype, int o_dtype,
                                       size_t capacity_pages);

/* ---- split-KV across GPUs without a collective library: peer-memory exchange + combine --
 * One kernel per step and rank: it stores this rank's (o, m, l) partial into every rank's
 * gather buffer over NVLink peer memory, publishes a per-rank flag, waits - bounded, about a
 * second, then MLC_DEVERR_WAIT_TIMEOUT in the device error word and no output - until all
 * ranks' partials of this step are in its own memory, and applies the combine rule of
 * mlc_encode_lse_combine. No counterpart in the reference (one device). Set-up, once:
 *   mlc_exchange_create   allocates this rank's gather buffer (cudaMalloc, zeroed)
 *   mlc_exchange_handle   64-byte cudaIpc handle of it; exchange the handles of all ranks by any
 *                         host channel (torch.distributed all_gather_object, a file, MPI ...)
 *   mlc_exchange_attach   handles = [world][MLC_IPC_HANDLE_BYTES], own entry ignored
 * Ranks are separate processes, one per GPU of one node; every rank must make the same sequence
 * of mlc_encode_exchange_lse_combine calls; synchronise the ranks on the host between the last
 * call's completion and mlc_exchange_destroy. Capturable in a CUDA graph (the step counter is
 * kept on the device). world <= 16, rows <= max_rows, head_dim % 4 == 0. */
#define MLC_IPC_HANDLE_BYTES 64
typedef struct mlc_exchange mlc_exchange;
int mlc_exchange_create(mlc_ctx* ctx, int rank, int world, size_t max_rows, size_t head_dim, mlc_exchange** out);
int mlc_exchange_handle(mlc_ctx* ctx, mlc_exchange* ex, void* handle_out);
int mlc_exchange_attach(mlc_ctx* ctx, mlc_exchange* ex, const void* handles);
/* The same for ranks that live in ONE process (one host thread and context per GPU, peer access
 * enabled by the caller): bases[r] = mlc_exchange_local_buffer of rank r's exchange object, own
 * entry ignored. Nothing is mapped or closed by the library. */
int mlc_exchange_attach_pointers(mlc_ctx* ctx, mlc_exchange* ex, void* const* bases);
void* mlc_exchange_local_buffer(const mlc_exchange* ex);
/* Profiling aid (context created with MLC_B200_TRACE=1): %globaltimer stamps, in ns, of CTA 0 of the
 * most recent exchange kernel: [0] start, [1] this rank's rows stored to a peer, [2] that peer's flag
 * stored, [3] every rank's flag seen, [4] combine done. */
int mlc_exchange_read_trace(mlc_ctx* ctx, unsigned long long* out8);
/* Floats per (step parity, rank) slot of the gather buffer: max_rows * (head_dim + 2) rounded up
 * to a multiple of 4, so that every slot starts on a 16-byte boundary. */
size_t mlc_exchange_slot_floats(const mlc_exchange* ex);
/* Layout of a rank's gather buffer (pure host arithmetic, no device needed): slots
 * [2 parities][world] of slot_floats floats each (o rows, then (m, l) pairs), flag words at
 * flags_offset bytes, behind them the stamped slots of the fused attention + exchange kernel
 * (every float beside a 4-byte step stamp), total size. Any output pointer may be null. */
int mlc_exchange_layout(int world, size_t max_rows, size_t head_dim, size_t* slot_floats,
                        size_t* flags_offset, size_t* total_bytes);
/* Partial attention over this rank's slice of the pages, the exchange and the combine as ONE launch:
 * the CTA that finishes a (request, head) stores its un-normalised rows straight into every rank's
 * gather buffer - every float beside the step's stamp in one 8-byte unit, so a row is complete when
 * its own bytes say so: no flag, no fence - then reads every rank's rows of that (request, head) from
 * its own memory, waiting - bounded, as above - for stamps that are not there yet, combines them and
 * writes `out` ([batch, num_heads, head_dim] of o_dtype, the full attention output, on every rank). `plan` covers this rank's slice (tables of its pages, the
 * tokens that fall into them, apply_causal 0 on all but the rank with the last tokens - as for
 * mlc_encode_paged_attention_partial_planned); every rank makes the same sequence of calls on an
 * exchange created for >= batch * num_heads rows. Plans the unit-mode kernel does not take fall back
 * to the partial + mlc_encode_exchange_lse_combine pair inside the call. Capturable. */
int mlc_encode_paged_attention_exchange_planned(mlc_ctx* ctx, const mlc_attn_plan* plan, mlc_exchange* ex,
                                                const void* q, const void* k_pages, const void* v_pages,
                                                void* out, float scale, int q_dtype, int o_dtype);
int mlc_encode_exchange_lse_combine(mlc_ctx* ctx, mlc_exchange* ex, const float* o_partial,
                                    const float* ml_partial, size_t rows, void* out, int o_dtype);
void mlc_exchange_destroy(mlc_ctx* ctx, mlc_exchange* ex);

/* ---- CUDA-graph bracketing of a pass --------------------------------------------------
 * Records the planned encode_* calls issued between begin and end into a CUDA graph
 * that replays them with one launch (the reference pays one command-buffer commit
 * per pass, metal_runtime.mm:6030-6033). Only the *_planned entry points and
 * mlc_encode_lse_combine may be called while capturing; run the same sequence once
 * outside a capture first so that workspaces exist. */
typedef struct mlc_graph mlc_graph;
int mlc_graph_begin_capture(mlc_ctx* ctx);
int mlc_graph_end_capture(mlc_ctx* ctx, mlc_graph** out);
int mlc_graph_launch(mlc_ctx* ctx, mlc_graph* graph);
void mlc_graph_destroy(mlc_ctx* ctx, mlc_graph* graph);

/* ======================================================================================
 * Host-side objects (C++17 inside the library, like the reference's): page allocator,
 * per-request page tables, per-layer paged storage, executor, scheduler.
 * int-returning functions in this part return 1 for "ok / has value" and 0 for the
 * reference's nullopt / false, unless they say mlc_status.
 * ====================================================================================== */

/* ---- PagePool (compiler/runtime/paged_kv.hpp:28-53, paged_kv.cpp:10-42): LIFO free list
 * of page ids; a fresh pool hands out 0, 1, 2, ...; allocate_n is all-or-nothing. */
typedef struct mlc_page_pool mlc_page_pool;
mlc_page_pool* mlc_page_pool_create(uint32_t capacity);
void mlc_page_pool_destroy(mlc_page_pool* pool);
int mlc_page_pool_allocate(mlc_page_pool* pool, uint32_t* page_id);
int mlc_page_pool_allocate_n(mlc_page_pool* pool, size_t n, uint32_t* out /* [n] */);
/* release: the reference asserts on a bad id (paged_kv.cpp:37-42); this returns 0 and
 * changes nothing. */
int mlc_page_pool_release(mlc_page_pool* pool, uint32_t page_id);
uint32_t mlc_page_pool_capacity(const mlc_page_pool* pool);
size_t mlc_page_pool_in_use(const mlc_page_pool* pool);
size_t mlc_page_pool_free(const mlc_page_pool* pool);

/* ---- RequestKVState (paged_kv.hpp:65-97, paged_kv.cpp:44-81) */
typedef struct mlc_kv_state mlc_kv_state;
mlc_kv_state* mlc_kv_state_create(uint32_t request_id, uint32_t page_size_tokens);
void mlc_kv_state_destroy(mlc_kv_state* state);
int mlc_kv_state_reserve(mlc_kv_state* state, mlc_page_pool* pool, size_t target_tokens);
int mlc_kv_state_extend_one_token(mlc_kv_state* state, mlc_page_pool* pool, uint32_t* page_id,
                                  uint32_t* slot_in_page);
int mlc_kv_state_locate(const mlc_kv_state* state, size_t pos, uint32_t* page_id, uint32_t* slot_in_page);
void mlc_kv_state_release_all(mlc_kv_state* state, mlc_page_pool* pool);
size_t mlc_kv_state_total_tokens(const mlc_kv_state* state);
uint32_t mlc_kv_state_tokens_in_last_page(const mlc_kv_state* state);
/* Copies up to `capacity` page ids; returns the table's length. */
size_t mlc_kv_state_page_table(const mlc_kv_state* state, uint32_t* out, size_t capacity);

/* ---- PagedKVStorage (paged_kv.hpp:109-145, paged_kv.cpp:83-127): one zero-filled K pool
 * and one V pool of capacity_pages * page_bytes per layer, owned by the object. */
typedef struct mlc_kv_storage mlc_kv_storage;
mlc_kv_storage* mlc_kv_storage_create(mlc_ctx* ctx, uint32_t capacity_pages, uint32_t n_layers,
                                      uint32_t page_size_tokens, uint32_t n_kv_heads, uint32_t head_dim,
                                      uint32_t dtype_bytes);
void mlc_kv_storage_destroy(mlc_kv_storage* storage);
int mlc_kv_storage_initialize(mlc_kv_storage* storage);
void* mlc_kv_storage_k_buffer(const mlc_kv_storage* storage, size_t layer);
void* mlc_kv_storage_v_buffer(const mlc_kv_storage* storage, size_t layer);
size_t mlc_kv_storage_page_bytes(const mlc_kv_storage* storage);

/* ---- executors (compiler/runtime/batched_executor.hpp:33-57: RequestSlot,
 * BatchedDecodeOutput, IBatchedExecutor) */
typedef struct mlc_request_slot {
    uint32_t request_id;
    uint64_t input_token;
    uint64_t sequence_position;
} mlc_request_slot;
typedef struct mlc_decode_row {      /* BatchedDecodeOutput::PerRequest */
    uint32_t request_id;
    int success;
    const float* logits;             /* valid until the callback is entered again */
    size_t n_logits;
} mlc_decode_row;
/* An IBatchedExecutor implemented by the caller (the seam the reference's scheduler tests
 * mock, tests/test_scheduler.cpp:22-60). run_decode fills rows[0..n) and returns how many
 * it filled; run_prefill returns the number of logits and points *logits at them. */
typedef struct mlc_executor_callbacks {
    void* user;
    size_t (*run_decode)(void* user, const mlc_request_slot* slots, size_t n, mlc_decode_row* rows);
    size_t (*run_prefill)(void* user, uint32_t request_id, const uint64_t* tokens, size_t n, const float** logits);
    void (*release_request)(void* user, uint32_t request_id);
} mlc_executor_callbacks;

typedef struct mlc_executor mlc_executor;
/* The paged-attention part of the reference's BatchedExecutor + BatchedWalker
 * (batched_executor.cpp:29-65, 96-103, 445-467; batched_walker.cpp:127-149, 299-331):
 * per-request page state, one batched pass = extend every request by one token, then per
 * layer write the new K/V rows and run attention. The model around attention is out of
 * scope: Q and the new K/V rows come from a deterministic hash of (seed, request, token,
 * position, layer) - see mlc_hash_qkv_value - and the "logits" are the last layer's
 * attention output, num_heads * head_dim floats per request. */
mlc_executor* mlc_paged_executor_create(mlc_ctx* ctx, uint32_t num_heads, uint32_t kv_heads, uint32_t head_dim,
                                        uint32_t n_layers, uint64_t qkv_seed);
mlc_executor* mlc_callback_executor_create(const mlc_executor_callbacks* callbacks);
/* A model for the paged executor: device-resident weights in the tensor roles the reference's
 * walker reads from the GGUF file (batched_walker.cpp:183-208 token_embd, :248-405 per layer
 * attn_norm / attn_qkv / attn_output / ffn_norm / ffn gate | up / ffn_down, :407-435 output_norm
 * and the lm_head). Norm weights are fp32 [hidden_size]; mat-vec weights and the token table are
 * Q4_0 rows, tightly packed; the lm_head is Q6_K (lm_head_quant = 1) or Q4_0 (0). hidden_size
 * must equal num_heads * head_dim and, like ffn_inner, be a multiple of 256.
 * With a model attached, mlc_executor_run_decode runs the whole walker step on the GPU and returns
 * vocab_size logits per request; in the fused call order (the default) a layer is 7 launches, in
 * the reference's call order (mlc_executor_set_call_order) the reference's 13, op for op. A prompt
 * (mlc_executor_run_prefill) is fed token by token through the decode path in the reference's call
 * order, as batched_executor.cpp:450-467 does, and 32 tokens per pass in the fused order; either
 * way the logits returned are the last prompt token's. The pointers must stay valid while the
 * executor lives. */
typedef struct mlc_layer_weights {
    const void* attn_norm;
    const void* attn_qkv;      /* [(num_heads + 2 kv_heads) * head_dim] rows of hidden_size */
    const void* attn_output;   /* [hidden_size] rows of hidden_size */
    const void* ffn_norm;
    const void* ffn_gate_up;   /* [2 * ffn_inner] rows of hidden_size: gate rows, then up rows */
    const void* ffn_down;      /* [hidden_size] rows of ffn_inner */
} mlc_layer_weights;
typedef struct mlc_model_desc {
    uint32_t hidden_size, ffn_inner, vocab_size, rotary_dim;
    float rope_base, rope_scale, rms_epsilon;
    int32_t lm_head_quant;
    const void* token_embd;    /* [vocab_size] Q4_0 rows of hidden_size */
    const void* output_norm;
    const void* lm_head;       /* [vocab_size] rows of hidden_size */
    const mlc_layer_weights* layers;
    uint32_t n_layers;
} mlc_model_desc;
int mlc_executor_attach_model(mlc_executor* exec, const mlc_model_desc* model);
/* ---- GGUF files (compiler/frontends/gguf_loader.{hpp,cpp}: GGUFLoader) -------------------------
 * The container the reference loads its models from, versions 1 to 3: header, typed key / value
 * metadata, tensor directory (sizes by ggml block format, offsets relative to the aligned end of the
 * directory, general.alignment honoured), tensor bytes read through a read-only mapping, and the
 * reference's byte-concatenation of every block's attn_q | attn_k | attn_v and ffn_gate | ffn_up
 * (Q4_0) into the fused attn_qkv and ffn_gate_up the batched walker multiplies with
 * (GGUFLoader::concatenateBlockWeights, gguf_loader.cpp:877-943). Version 1 is read as the reference
 * reads it (and its tests write it): 32-bit tensor dimensions, optionally behind a 64-bit repeat of the
 * rank, offsets that are file positions. A key longer than 1 MiB is dropped with its value
 * (gguf_loader.cpp:553-607); damaged files the reference's other recovery heuristics would read on
 * through are rejected with a message.
 * Functions that can fail take an optional `error` buffer for the message (always terminated).
 *   mlc_gguf_open                     GGUFLoader(path) + load(); NULL on failure
 *   mlc_gguf_concatenate_block_weights  number of tensors added, -1 on failure
 *   mlc_gguf_describe                 everything but the tensor bytes as one JSON object
 *                                     {version, n_tensors, n_kv, alignment, data_start,
 *                                      quantization_version, kv: {key: {type, [elem_type,] value}},
 *                                      tensors: {name: {shape, dtype, offset (absolute; -1 for a
 *                                      concatenated tensor), n_bytes}}}; returns the bytes needed
 *                                     including the terminator, copies at most `capacity`
 *   mlc_gguf_tensor_data              GGUFLoader::loadTensorData: copies min(capacity, n_bytes) bytes
 *                                     (dst may be NULL) and returns n_bytes, -1 on failure
 *   mlc_executor_attach_gguf          reads the decoder out of the file - token_embd, per block
 *                                     attn_norm, attn_qkv, attn_output, ffn_norm, ffn_gate_up, ffn_down,
 *                                     output_norm, output (or the embedding table when the file ties
 *                                     them), sizes and rotary / norm constants from the llama.* keys -
 *                                     uploads the weights into one device allocation the executor owns
 *                                     and attaches them like mlc_executor_attach_model. mlc_status. */
typedef struct mlc_gguf mlc_gguf;
mlc_gguf* mlc_gguf_open(const char* path, char* error, size_t error_capacity);
void mlc_gguf_close(mlc_gguf* file);
int mlc_gguf_concatenate_block_weights(mlc_gguf* file, char* error, size_t error_capacity);
size_t mlc_gguf_describe(mlc_gguf* file, char* json, size_t capacity);
int64_t mlc_gguf_tensor_data(mlc_gguf* file, const char* name, void* dst, size_t capacity, char* error,
                             size_t error_capacity);
int mlc_executor_attach_gguf(mlc_executor* exec, mlc_gguf* file, char* error, size_t error_capacity);

/* ---- Tokenizer (compiler/runtime/tokenizer.{hpp,cpp}: Tokenizer, as built without llama.cpp) -------
 * Text <-> token ids from the vocabulary of a GGUF file (tokenizer.ggml.model / tokens / scores / merges /
 * bos_token_id / eos_token_id / unk_token_id): best-score segmentation for "llama" / "spm" / "unigram"
 * vocabularies, lowest-rank-first byte-pair merges for "gpt2" / "bpe" (and for a file with merges and no
 * model key), longest-match when neither produced anything and no BOS was put in front; "<0xHH>" pieces
 * are bytes. Same results as the reference's own code paths (tokenizer.cpp:153-244, 246-283, 327-423) on
 * the same file and text; its optional llama.cpp path is not reproduced.
 *   mlc_tokenizer_create        Tokenizer(loader); the file may be closed afterwards
 *   mlc_tokenizer_info          returns valid(); vocabSize(), bosId(), eosId(), unkId() (UINT64_MAX = unset)
 *   mlc_tokenizer_encode        encode(text, {add_bos, add_eos}): returns the number of ids, copies at
 *                               most `capacity`
 *   mlc_tokenizer_decode        decode(ids): returns the number of bytes, copies at most `capacity`
 *                               (no terminator)
 *   mlc_tokenizer_token_string  tokenString(id), same convention
 *   mlc_tokenizer_token_flags   bit 0 isControlToken(id), bit 1 isEogToken(id) */
typedef struct mlc_tokenizer mlc_tokenizer;
mlc_tokenizer* mlc_tokenizer_create(mlc_gguf* file);
void mlc_tokenizer_destroy(mlc_tokenizer* tokenizer);
int mlc_tokenizer_info(const mlc_tokenizer* tokenizer, size_t* vocab_size, uint64_t* bos, uint64_t* eos, uint64_t* unk);
size_t mlc_tokenizer_encode(const mlc_tokenizer* tokenizer, const char* text, size_t length, int add_bos, int add_eos,
                            uint64_t* ids, size_t capacity);
size_t mlc_tokenizer_decode(const mlc_tokenizer* tokenizer, const uint64_t* ids, size_t n, char* out, size_t capacity);
size_t mlc_tokenizer_token_string(const mlc_tokenizer* tokenizer, uint64_t id, char* out, size_t capacity);
int mlc_tokenizer_token_flags(const mlc_tokenizer* tokenizer, uint64_t id);

/* No counterpart in the reference. Gives a request without pages a context of `tokens` tokens whose
 * K/V rows the caller has put (or will put) into the storage itself: reserves its pages
 * (RequestKVState::reserve) and sets its next position to `tokens`. For restoring a saved context and
 * for benchmarks that start from long contexts. MLC_ERR_INVALID_ARG if the request already has pages
 * or the pool cannot supply them. */
int mlc_executor_assume_context(mlc_executor* exec, uint32_t request_id, size_t tokens);

void mlc_executor_destroy(mlc_executor* exec);
/* attach_page_pool / attach_paged_storage (batched_executor.hpp:73, 90); mlc_status. */
int mlc_executor_attach_page_pool(mlc_executor* exec, mlc_page_pool* pool, uint32_t page_size_tokens);
int mlc_executor_attach_paged_storage(mlc_executor* exec, mlc_kv_storage* storage);
/* 0 (default): one fused launch per layer; 1: the reference's order - scatter K, scatter V,
 * attention with host tables per layer (batched_walker.cpp:299-331). mlc_status. */
int mlc_executor_set_call_order(mlc_executor* exec, int reference_order);
/* run_decode: returns the number of per-request results; success[i] and, for successful
 * requests, logits[i * logits_stride ...] are filled. With a model attached and logits_stride >=
 * vocab_size the rows are written without intermediate per-request vectors - straight from the
 * device when `logits` is page-locked host memory (cudaHostAlloc / cudaHostRegister / pin_memory). */
size_t mlc_executor_run_decode(mlc_executor* exec, const mlc_request_slot* slots, size_t n, uint8_t* success,
                               float* logits, size_t logits_stride);
/* The same pass ending in greedy sampling on the device (model attached, fused call order): tokens[i] =
 * index of the first maximum of slot i's logits, UINT64_MAX for a slot that failed; 128 bytes cross the bus
 * instead of batch * vocab_size floats. Returns n, or 0 when the executor cannot do it (nothing has run
 * then: use mlc_executor_run_decode). The scheduler uses this path by itself. */
size_t mlc_executor_run_decode_greedy(mlc_executor* exec, const mlc_request_slot* slots, size_t n, uint64_t* tokens);
/* run_prefill: returns the number of logits (0 = failed). */
size_t mlc_executor_run_prefill(mlc_executor* exec, uint32_t request_id, const uint64_t* tokens, size_t n,
                                float* logits, size_t capacity);
void mlc_executor_release_request(mlc_executor* exec, uint32_t request_id);
size_t mlc_executor_live_request_count(const mlc_executor* exec);
size_t mlc_executor_known_position(const mlc_executor* exec, uint32_t request_id);
/* page_state() (batched_executor.hpp:77): copies the request's page ids, returns their count. */
size_t mlc_executor_page_table(const mlc_executor* exec, uint32_t request_id, uint32_t* out, size_t capacity,
                               size_t* total_tokens);
/* Element `index` of tensor 0 (Q), 1 (K row) or 2 (V row) the paged executor feeds. */
float mlc_hash_qkv_value(uint64_t seed, uint32_t request, uint64_t token, uint64_t position, uint32_t layer,
                         uint32_t tensor, uint32_t index);

/* ---- Scheduler (compiler/runtime/scheduler.hpp:27-104, scheduler.cpp:10-186) */
typedef struct mlc_scheduler mlc_scheduler;
typedef void (*mlc_token_callback)(void* user, uint32_t request_id, uint64_t token);
mlc_scheduler* mlc_scheduler_create(mlc_executor* exec, size_t max_batch_size /* reference default 8 */);
void mlc_scheduler_destroy(mlc_scheduler* sched);
uint32_t mlc_scheduler_add_request(mlc_scheduler* sched, const uint64_t* prompt_tokens, size_t n,
                                   size_t max_new_tokens /* reference default 100 */,
                                   int64_t eos_token_id /* -1 disables */);
void mlc_scheduler_set_token_callback(mlc_scheduler* sched, mlc_token_callback cb, void* user);
/* Chunked admission (an addition: the reference feeds a prompt whole in one tick, scheduler.cpp:47-81):
 * a prompt is fed at most `tokens` at a time, one chunk per tick, the batch's decode pass running every
 * tick in between. 0 = whole prompts. mlc_scheduler_prefill_calls counts the run_prefill calls made. */
void mlc_scheduler_set_prefill_chunk_tokens(mlc_scheduler* sched, size_t tokens);
size_t mlc_scheduler_prefill_calls(const mlc_scheduler* sched);
int mlc_scheduler_tick(mlc_scheduler* sched);
size_t mlc_scheduler_run_until_idle(mlc_scheduler* sched);
int mlc_scheduler_empty(const mlc_scheduler* sched);
size_t mlc_scheduler_queued_count(const mlc_scheduler* sched);
size_t mlc_scheduler_active_count(const mlc_scheduler* sched);
size_t mlc_scheduler_completed_count(const mlc_scheduler* sched);
void mlc_scheduler_stats(const mlc_scheduler* sched, size_t* requests_completed, size_t* decode_steps,
                         size_t* tokens_generated);
/* drain_completed(): moves the completed requests into the handle and returns their count;
 * mlc_scheduler_drained_request reads one of them (state: 0 Queued, 1 Prefilling, 2 Decoding,
 * 3 Complete, 4 Failed). */
size_t mlc_scheduler_drain_completed(mlc_scheduler* sched);
int mlc_scheduler_drained_request(const mlc_scheduler* sched, size_t index, uint32_t* id, int* state,
                                  size_t* n_generated, uint64_t* generated, size_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* MLC_B200_H */
