// Shared declarations of the attention entry points and their two kernel families.
#pragma once

#include "ctx.hpp"

struct mlc_attn_plan;
struct mlc_ctx;

namespace mlcb {

// One attention call after validation (host arrays already checked).
struct AttnArgs {
    const void* q = nullptr;
    const void* k_pages = nullptr;
    const void* v_pages = nullptr;
    void* o = nullptr;
    size_t batch = 0, H = 0, KVH = 0, D = 0, P = 0;
    size_t capacity = 0;  // pages in the pool, 0 = unknown
    float scale = 0.f;
    int q_dtype = MLC_F32, o_dtype = MLC_F32;
    // Split-KV partial output (un-normalised o + (m, l) per row) instead of O.
    float* o_partial = nullptr;
    float* ml_partial = nullptr;
    // Decode step: this step's new rows, fp16 [batch, KVH, D]; written into the pools by
    // the attention kernel itself (the pools are then written to, not only read).
    const void* k_new = nullptr;
    const void* v_new = nullptr;
    // The kernel in front wrote nothing into the pools but the rows at the plan's (page, slot) per request - the
    // newest token of every request (a step-fusable plan marks the tiles that hold them): every other tile may be
    // fetched before the wait for that kernel, as in a decode step. Not for prompt chunks, whose rows land in tiles
    // that other entries of the batch read.
    bool only_plan_rows_written = false;
    // Caller-provided split-KV workspace (device memory) instead of the context's own;
    // when set, the launch makes no device or host allocation at all.
    void* ext_work = nullptr;
    size_t ext_work_bytes = 0;
    // Fused exchange across GPUs (unit-mode plans): finished rows go to every rank's gather buffer, this rank
    // combines all ranks' rows into exchange_out (of o_dtype). q / o above are not used for output then.
    const ExchangeView* exchange = nullptr;
    void* exchange_out = nullptr;
};

// ---- work plan of the TMA / tensor-core kernel ----------------------------------
// The kernel is persistent: CTA c owns a contiguous range of "tiles" in the order
// (request, head block, tile), a tile being kTileTokens consecutive tokens of one
// request for the kDecodeWarps KV heads of one head block. A maximal run of tiles
// with the same (request, head block) inside a CTA's range is a piece; a (request,
// head block) whose tiles span several CTAs is a split segment, whose pieces are
// merged by a second, tiny kernel.
static constexpr int kDecodeWarps = 4;   // KV heads per head block = warps per CTA
static constexpr int kTileTokens = 32;   // tokens per pipeline stage
// Warps of a CTA in unit mode: with one KV head per CTA a warp's tile costs ~0.8 us of dependent
// work, so the longest (request, head) is cut into more parts where shared memory allows.
#ifndef MLCB_UNIT_WARPS_D64
#define MLCB_UNIT_WARPS_D64 8
#endif
constexpr int unit_warps(size_t head_dim) { return head_dim == 64 ? MLCB_UNIT_WARPS_D64 : 4; }
// Tile word: page id | sub-tile within the page | head block | "holds this step's new token".
static constexpr uint32_t kTilePageMask = (1u << 22) - 1;
static constexpr uint32_t kTileSubShift = 22;
static constexpr uint32_t kTileHbShift = 25;
static constexpr uint32_t kTileHbMask = 0x3Fu;
static constexpr uint32_t kTileFreshBit = 1u << 31;

struct PieceDesc {
    uint32_t req;
    uint32_t tile_begin;      // first tile of the piece, in tiles from the request's token 0
    uint32_t n_tiles;
    uint32_t part_slot;       // workspace slot this piece writes when n_parts > 1
    uint32_t seg_first_slot;  // first workspace slot of the (request, head block) segment
    uint32_t seg;             // index of the split segment (0 when not split)
    uint16_t n_parts;         // pieces the segment is split into (1: write O directly)
    uint16_t hb;              // head block: KV heads hb*kDecodeWarps ...
    uint16_t last_valid;      // valid tokens in the piece's last tile, 1..kTileTokens
    uint16_t flags;           // bit 0: the piece's last tile ends with the request's newest token
};
static_assert(sizeof(PieceDesc) == 32, "PieceDesc is read as two 16-byte vectors");

struct SegDesc {              // one split (request, head block): input of the merge kernel
    uint32_t req, hb, first_slot, n_parts;
};

struct DecodePlanView {            // device addresses inside one plan blob
    const uint32_t* cta_counts;    // [n_cta][2] = {pieces, tiles}
    const PieceDesc* pieces;       // [n_cta][max_pieces]
    const uint32_t* tile_pages;    // [n_cta][max_tiles] page id of every tile
    const uint32_t* pt_flat;       // copies of the caller's tables (general kernel, checks)
    const uint32_t* pt_off;
    const uint32_t* eff_len;       // tokens each request attends to
    const uint32_t* zero_rows;     // requests with eff_len == 0 (their O rows are zero-filled)
    const SegDesc* seg_desc;       // [n_segs] split segments
    bool has_tma = false;          // the per-CTA tile lists above were built
    bool step_fusable = false;     // every request's newest token is the last one it attends to
    bool unit_mode = false;        // per-warp plan slices, no request split over CTAs (see the kernel)
    uint32_t stages = 3;           // ring depth the plan was cut for
    uint32_t n_cta = 0, max_pieces = 0, max_tiles = 0, n_zero = 0;
    uint32_t n_slots = 0, n_segs = 0;
    uint32_t n_unit_cuts = 0;      // unit mode: (request, head) units cut over CTAs, one arrival counter each
    uint32_t hpc = 1;              // unit mode: KV heads a CTA works on at a time (see DecodeParams::hpc)
    bool pass_ready = false;       // this view was laid out for whole-pass launches
};

int launch_attention_general(mlc_ctx* ctx, const AttnArgs& a, const uint32_t* d_pt_flat,
                             const uint32_t* d_pt_off, const uint32_t* d_eff_len);

// True when the TMA / tensor-core kernel covers this shape / these pointers.
bool decode_tma_shape_supported(size_t H, size_t KVH, size_t D, size_t P, size_t capacity);
bool decode_tma_pointers_supported(const AttnArgs& a);
// Deepest TMA ring that fits in shared memory next to the kernel's merge buffers.
uint32_t decode_tma_max_stages(size_t H, size_t KVH, size_t D);
size_t decode_tma_smem_bytes(size_t D, bool g16, uint32_t stages, bool unit);
// One launch writing this step's K and V rows; page ids and slots already on the device.
int launch_scatter_rows_device_tables(mlc_ctx* ctx, void* k_pool, void* v_pool, const uint32_t* d_ids,
                                      const uint32_t* d_slots, size_t P, size_t KVH, size_t D,
                                      size_t batch, const void* k_src, const void* v_src, size_t capacity);
int launch_attention_decode_tma(mlc_ctx* ctx, const AttnArgs& a, const DecodePlanView& plan);
int encode_attention_planned_after_row_write(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q, const void* k_pages,
                                             const void* v_pages, void* o, float scale, int q_dtype, int o_dtype);
// Whole-pass launch: every layer's decode step (row write + attention) in one kernel. `shape` carries the
// plan's shape, scale and dtypes. MLC_ERR_UNSUPPORTED (without an error text) when a layer's pointers do not
// meet the TMA kernel's alignment rules: the caller then launches layer by layer.
bool decode_pass_supported(const DecodePlanView& plan, size_t n_layers);
int launch_decode_pass_tma(mlc_ctx* ctx, const AttnArgs& shape, const DecodePlanView& plan, size_t n_layers,
                           const void* const* q, const void* const* k_new, const void* const* v_new,
                           void* const* k_pages, void* const* v_pages, void* const* o);

// Chunked causal prefill on tcgen05 (attn_prefill_tcgen05.cu): D = 128, 64-token pages, fp16 q / o.
bool prefill_tcgen05_supported(size_t H, size_t KVH, size_t D, size_t P, size_t capacity);
int launch_prefill_tcgen05(mlc_ctx* ctx, const void* q, const void* k_pages, const void* v_pages, void* o,
                           const uint32_t* d_pt_flat, const uint32_t* d_pt_off, const uint32_t* d_seq_lens,
                           const uint32_t* d_q_start, const uint32_t* d_q_len, const uint32_t* d_q_row0,
                           size_t batch, size_t total_q, size_t max_q_len, size_t H, size_t KVH, size_t capacity,
                           float scale);
// Launches attention for an already created plan (the plan's shape fields fill `a`).
int launch_attention_with_plan(mlc_ctx* ctx, AttnArgs a, const mlc_attn_plan* plan);

// Before a launch that reads a plan's device copy: waits for an upload that went to the copy stream and notes
// the use (attn_api.cu).
int use_plan(mlc_ctx* ctx, const mlc_attn_plan* plan);

}  // namespace mlcb
