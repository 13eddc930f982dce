// Host-side launch functions of the verify-step kernels (definitions in the .cu files beside this one).
#pragma once

#include "common.cuh"
#include "tma.cuh"

namespace ei {

// Device-resident state of one session: what the captured step reads instead of host values
// (generalises the reference's graph control block, runtime/src/qwen3.cpp:66-72).
struct Control {
  int32_t context;    // committed KV rows; the step's first row goes to this position
  uint32_t pending;   // last emitted token = row 0 of the next step
  int32_t status;     // 0 ok; bit 0: step would exceed capacity (step skipped); bit 1: bad token id
  int32_t steps;      // verify steps executed since the last drain
  unsigned long long emitted_total;  // tokens emitted since the last drain
  ei_verify_result last;
};

// One session of a wide batch (more than 16 stacked rows): where its device state lives. Kernels of the wide
// step take an array of these and find their session from the stacked row (or a grid dimension).
struct SessionSlot {
  Control* control;
  bf16* k_cache;  // layer 0; layer l at k_cache + l * capacity * kv_heads * 128
  bf16* v_cache;
  int capacity;
  int reserved;
};

// ---- elementwise.cu ----
void launch_rms_norm(const bf16* in, const bf16* weight, bf16* out, size_t rows, size_t width, float eps,
                     cudaStream_t stream, bool pdl);
void launch_add(const bf16* a, const bf16* b, bf16* out, size_t count, int multiprocessors, cudaStream_t stream);
void launch_silu_multiply(const bf16* gate, const bf16* up, bf16* out, size_t count, int multiprocessors,
                          cudaStream_t stream);
void launch_gather(const uint32_t* ids, const bf16* table, bf16* out, size_t rows, size_t width,
                   size_t vocabulary, int multiprocessors, cudaStream_t stream);
void launch_rope(bf16* data, size_t rows, size_t heads, size_t head_dim, size_t row_stride,
                 const float* table, size_t table_stride, size_t offset, const size_t* offsets,
                 const int* pingpong, int multiprocessors, cudaStream_t stream);
void launch_store_kv(const bf16* source, bf16* cache, size_t rows, size_t width, size_t capacity,
                     size_t offset, const size_t* device_offset, int multiprocessors, cudaStream_t stream);

// Device-resident description of a draft array: drafts[position - base] is the token proposed for
// absolute position `position`. Read at kernel time so a captured graph follows a change of array.
struct DraftSource {
  const uint32_t* drafts;
  long long base, count;
};

// Device-resident description of where a session records what it emits: tokens[position - base] receives the
// token emitted for absolute position `position` (the token after the first `position` ones). Read at kernel
// time. A draft session's sink is the array the target session takes its drafts from.
struct TokenSink {
  uint32_t* tokens;
  long long base, count;
};

struct EmbedParams {
  const uint32_t* tokens;     // host-driven step: [rows] device tokens; null in the device-resident loop
  const DraftSource* source;  // device-resident loop: row 0 = control->pending, row i = draft of position context + i
  Control* control;
  uint32_t* step_tokens;    // [rows] out: the tokens this step consumed (inputs of the acceptance)
  const bf16* table;        // [vocab, hidden]
  int vocab, hidden, rows, capacity;
  const bf16* norm_weight;
  float eps;
  bf16* residual;           // [rows, hidden]
  bf16* normed;             // [rows, hidden]
  const SessionSlot* slots; // wide batch: stacked row r belongs to session r / rows_per_session (control and
  int rows_per_session;     // capacity above are then unused; rows = all stacked rows; tokens must be given)
};
// Token selection + embedding lookup + first RMSNorm, one block per row.
void launch_embed_norm(const EmbedParams& p, cudaStream_t stream, bool pdl);

struct QkvParams {
  bf16* qkv;                // [rows, (heads + 2 kv_heads) * 128] : q | k | v, q and k rotated in place
  int rows, heads, kv_heads, qkv_stride;
  const bf16* q_norm;       // [128] or null
  const bf16* k_norm;
  float eps;
  const float* rope_table;  // [max_pos, 128]
  int max_positions;
  const Control* control;
  int capacity;
  bf16* k_cache;            // [capacity, kv_heads * 128] of this layer
  bf16* v_cache;
  const SessionSlot* slots; // wide batch, as in EmbedParams; the caches are the slots' at `layer`
  int rows_per_session, layer;
};
// Per-head QK RMSNorm + RoPE + KV append at the device-side context length, one warp per (row, head).
void launch_qk_norm_rope_store(const QkvParams& p, cudaStream_t stream, bool pdl);

struct ResidualNormParams {
  const float* partial;     // [ksplit, rows, hidden] FP32 partial sums of the projection
  int ksplit, rows, hidden;
  const bf16* bias;         // projection bias or null
  bf16* residual;           // in/out
  const bf16* norm_weight;  // weight of the RMSNorm that follows
  float eps;
  bf16* normed;             // out
};
// projection = round(sum partial + bias); residual = round(residual + projection); normed = RMSNorm(residual).
void launch_residual_norm(const ResidualNormParams& p, cudaStream_t stream, bool pdl);

// ---- attention.cu ----
struct AttentionParams {
  const bf16* q;            // row r, head h at q + r * q_stride + h * 128
  int q_stride;
  const bf16* k;            // token t, kv head j at k + t * kv_stride + j * 128
  const bf16* v;
  int kv_stride;
  int rows, heads, kv_heads;
  int capacity;             // tokens addressable in k / v
  const int32_t* device_offset;  // position of query row 0 (device) or null -> host_offset
  int host_offset;
  int chunk;                // tokens per split (multiple of 64)
  int max_splits;
  float* scratch;           // [max_splits][rows * heads][132]
  bf16* out;                // row r, head h at out + r * out_stride + h * 128
  int out_stride;
  const SessionSlot* slots; // wide batch: one grid slice per session (`sessions` of them), `rows` query rows
  int sessions, layer;      // each; session j reads q + j * rows * q_stride, its own cache and context length,
  size_t scratch_stride;    // scratch + j * scratch_stride (floats), and writes out + j * rows * out_stride
  // K / V tiles are fetched by TMA. A single session's maps are encoded by the launch function from k, v,
  // kv_stride, kv_heads and capacity; a wide batch passes one pair per session in device memory, built with
  // encode_kv_map over all layers of the session's cache (`layer` selects the slice).
  CUtensorMap k_map, v_map;
  const CUtensorMap* maps;  // [sessions][2] = (K, V)
  int* status;              // optional device word; bit 2 is set if a bounded wait on a copy gave up
  uint32_t wait_limit;      // polls before a bounded wait gives up (0: the default)
  uint32_t fault_tx;        // test hook: bytes the first copy is expected to deliver beyond what it does (0 in production)
};
// Tensor map of a K or V cache: bf16 [layers][tokens][kv_heads * 128] with `token_stride` elements between tokens
// and `layer_stride` between layers, described to TMA as (64 values, token, half of a head, kv head, layer) so
// that a 64-token tile of one head lands as [half][token][128 B] with the 128-byte swizzle.
void encode_kv_map(CUtensorMap* map, const bf16* base, size_t tokens, size_t token_stride, int kv_heads, size_t layers,
                   size_t layer_stride);
int attention_chunk_for(size_t kv_length);
size_t attention_scratch_bytes(size_t rows, size_t heads, size_t kv_length);
void launch_verify_attention(const AttentionParams& p, cudaStream_t stream, bool pdl);
// Any number of query rows in one launch, 16 per block over their whole causal history; no scratch, no merge
// (chunk, max_splits and scratch are not used).
void launch_prompt_attention(const AttentionParams& p, cudaStream_t stream, bool pdl);

// ---- sampling.cu ----
// Per-row argmax partials of logits [rows, vocab] into best_value / best_index [blocks, 16]; at most
// kSampleMaxParts blocks (the size every partial buffer is given).
constexpr int kSampleMaxParts = 256;
int sample_partial_blocks(size_t vocabulary, int multiprocessors);
void launch_argmax_partials(const bf16* logits, size_t rows, size_t vocab, size_t row_stride,
                            float* best_value, int* best_index, int blocks, cudaStream_t stream, bool pdl);
// Final argmax over `parts` partials per row; writes targets[rows]. With `control` non-null also
// performs greedy acceptance against step_tokens and commits the context length.
void launch_finalize(const float* best_value, const int* best_index, int parts, int rows,
                     uint32_t* targets, const uint32_t* step_tokens, Control* control,
                     int32_t* context_length, uint32_t* pending, ei_verify_result* result,
                     cudaStream_t stream, bool pdl, const TokenSink* sink = nullptr);
// Makes a draft session continue from where the target session stands: copies context length and pending token
// and inherits a raised status. One thread.
void launch_adopt_control(Control* mine, const Control* theirs, cudaStream_t stream);
// Wide batch: per-row argmax partials laid out [row][parts] for any number of rows, then per session the final
// argmax of its rows, acceptance against step_tokens and commit in its slot's control block.
void launch_argmax_partials_wide(const bf16* logits, size_t rows, size_t vocab, size_t row_stride, float* best_value,
                                 int* best_index, int parts, cudaStream_t stream, bool pdl);
void launch_finalize_wide(const float* best_value, const int* best_index, int parts, int rows_per_session,
                          int sessions, uint32_t* targets, const uint32_t* step_tokens, const SessionSlot* slots,
                          cudaStream_t stream, bool pdl);

// Acceptance only, from targets already chosen.
void launch_accept(const uint32_t* inputs, const uint32_t* targets, int rows, int32_t* context_length,
                   uint32_t* pending, ei_verify_result* result, cudaStream_t stream);

}  // namespace ei
