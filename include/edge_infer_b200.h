/* edge_infer_b200 - C ABI of the B200 (sm_100a) speculative-decoding verify step.
 *
 * Drop-in boundary for edge-infer's direct-operator API (namespace op::cuda) and its
 * runtime Session contract, for the BF16 / AWQ-int4 verify path only. Every entry point
 * is `extern "C"`, takes plain pointers, sizes and POD structs, allocates nothing unless
 * its comment says so, launches on the caller's stream and returns an ei_status.
 * "ref:" names the reference interface an entry point replaces
 * (paths relative to the edge-infer source tree).
 *
 * Element type: BF16 (`uint16_t` payload / __nv_bfloat16). Strides are in elements.
 */
#ifndef EDGE_INFER_B200_H
#define EDGE_INFER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. The reference throws C++ exceptions (ref: operators/src/cuda/execution.cu:15-58,
 * runtime/src/qwen3.cpp:127-161); each code names the exception type it stands for. */
typedef enum ei_status {
  EI_OK = 0,
  EI_INVALID_ARGUMENT = 1, /* std::invalid_argument */
  EI_OUT_OF_RANGE = 2,     /* std::out_of_range     */
  EI_OVERFLOW = 3,         /* std::overflow_error   */
  EI_RUNTIME = 4,          /* std::runtime_error (CUDA failure) */
  EI_LOGIC = 5,            /* std::logic_error      */
  EI_LENGTH = 6,           /* std::length_error     */
  EI_POISONED = 7          /* session unusable after a failed stream completion */
} ei_status;

/* Message of the calling thread's last failed call (valid until its next call). */
const char* ei_last_error(void);
/* Library version string. */
const char* ei_version(void);

/* ---- borrowed views; layout-identical to the reference's aggregates ----------------------
 * ref: core/include/tensor_view.hpp:18-26 (TensorView<T,Rank>{T* data; size_t shape[R]; size_t stride[R]})
 * ref: operators/include/operators/core/array_view.hpp:8-17 (ArrayView<T>{T* data; size_t size}) */
typedef struct ei_view1 { void* data; size_t shape[1]; size_t stride[1]; } ei_view1;
typedef struct ei_view2 { void* data; size_t shape[2]; size_t stride[2]; } ei_view2;
typedef struct ei_view3 { void* data; size_t shape[3]; size_t stride[3]; } ei_view3;
typedef struct ei_array { void* data; size_t size; } ei_array;

/* ref: operators/include/operators/cuda/execution.hpp:18-26 (ExecutionContext). `handle` is kept for
 * layout familiarity and ignored: no entry point calls cuBLAS. */
typedef struct ei_context {
  void* handle;
  void* stream; /* cudaStream_t */
  int32_t device;
  int32_t multiprocessors;
  int32_t max_threads_per_block;
  size_t shared_memory_limit;  /* opt-in maximum dynamic shared memory per block */
} ei_context;

/* ref: execution.hpp:34-41 (DenseLinearWeight<T>); operation: 1 = transposed storage
 * (each output's inputs contiguous, CUBLAS_OP_T), 0 = row-major [in, out] (CUBLAS_OP_N). */
typedef struct ei_dense_weight {
  const void* data;
  const void* bias;
  int32_t input_features, output_features, leading_dimension, operation;
} ei_dense_weight;

/* ref: execution.hpp:44-53 (AwqLinearWeight<T>): qweight int32 [N, K/8] with nibble k%8 at bit
 * 4*(k%8); scales BF16 [N, padded_groups]; zeros int32 [N, ceil(K/group/8)]. */
typedef struct ei_awq_weight {
  const int32_t* qweight;
  const void* scales;
  const int32_t* zeros;
  const void* bias;
  int32_t input_features, output_features, group_size, padded_groups;
} ei_awq_weight;

/* ---- context ---------------------------------------------------------------------------- */
/* ref: execution.hpp:28-29 prepare_execution_context(handle, stream); queries the current device. */
ei_status ei_prepare_execution_context(void* stream, ei_context* out);

/* ---- linear operators --------------------------------------------------------------------- */
/* ref: execution.hpp:55-57, execution.cu:267-284 prepare_dense<T>(weight [in,out] view, bias). */
ei_status ei_prepare_dense_bf16(ei_view2 weight, ei_view1 bias, ei_dense_weight* out);
/* ref: execution.hpp:58-64, execution.cu:285-298 prepare_awq<T>(qweight, scales, zeros, group, in, bias). */
ei_status ei_prepare_awq_bf16(ei_view2 qweight, ei_view2 scales, ei_view2 zeros, size_t group_size,
                              size_t input_features, ei_view1 bias, ei_awq_weight* out);
/* Bytes of caller-owned FP32 scratch the linear operators can use for `rows` input rows: partial sums of the
 * slices when the input features are split over blocks. Without scratch the operators still work; shapes that
 * need the split then take a slower kernel (<= 32 rows) or leave SMs idle (more rows, few output features). */
size_t ei_linear_scratch_bytes(size_t rows, size_t input_features, size_t output_features);
/* ref: execution.hpp:65-67, execution.cu:299-324 linear<T>: out[rows,N] = round_bf16(x W + bias), FP32
 * accumulation, bias added before the single rounding. rows <= 16 takes the streaming kernel;
 * more rows are processed 16 at a time. */
ei_status ei_linear_bf16(const ei_context* ctx, ei_view2 input, const ei_dense_weight* weight,
                         ei_view2 output, void* scratch, size_t scratch_bytes);
/* ref: execution.hpp:68-70, execution.cu:325-335, kernels/awq_gemv_gemm.cu:607-654 awq_linear<T>.
 * Dequantised weights are rounded to BF16 before the product, as the reference does for rows > 1
 * (awq_gemv_gemm.cu:119-127, 599); rows == 1 uses the same rule. */
ei_status ei_awq_linear_bf16(const ei_context* ctx, ei_view2 input, const ei_awq_weight* weight,
                             ei_view2 output, void* scratch, size_t scratch_bytes);

/* Fused SwiGLU projection, the step's largest kernel: `weight` holds the gate rows followed by the up rows
 * ([2F, K]; bias, if any, [2F]); out[rows, F] = round(round(silu(round(gate))) * round(up)).
 * ref: the reference issues two awq_linear calls and silu_multiply (runtime/include/execution/decoder.hpp:162-165,
 * operators/src/cuda/silu_cuda.cu:45-56); every rounding point of that sequence is kept. rows <= 16,
 * group_size 128, K % 256 == 0, F % 8 == 0. */
ei_status ei_awq_gate_up_silu_bf16(const ei_context* ctx, ei_view2 input, const ei_awq_weight* weight,
                                   ei_view2 output);

/* ---- element-wise / normalisation ------------------------------------------------------------- */
/* ref: execution.hpp:72-74, add_cuda.cu:144-180 add<T>. */
ei_status ei_add_bf16(const ei_context* ctx, ei_array a, ei_array b, ei_array out);
/* ref: direct.hpp:36-40, silu_cuda.cu:45-56 silu_multiply<T>: round(round(silu(g)) * u). */
ei_status ei_silu_multiply_bf16(const ei_context* ctx, ei_array gate, ei_array up, ei_array out);
/* ref: execution.hpp:87-92, rms_norm_cuda.cu:20-139 rms_norm<T>; 1 <= features <= 10240. */
ei_status ei_rms_norm_bf16(const ei_context* ctx, ei_array input, ei_array weight, ei_array out,
                           size_t rows, size_t features, float epsilon);
/* ref: execution.hpp:94-96, execution.cu:337-348 gather<T> (token >= vocabulary -> zeros). */
ei_status ei_gather_bf16(const ei_context* ctx, ei_view1 ids, ei_view2 table, ei_view2 out);
/* ref: execution.hpp:100-105, execution.cu:360-373 rope_precomputed<T>: table float [max_pos, head_dim]
 * with [2i] = sin, [2i+1] = cos; position = row + (offsets ? offsets[pingpong ? *pingpong : 0] : offset). */
ei_status ei_rope_precomputed_bf16(const ei_context* ctx, ei_view3 input, ei_view2 table, size_t offset,
                                   const size_t* offsets, const int* pingpong);
/* Builds that table on the host exactly as the reference's prepared model does.
 * ref: runtime/include/models/qwen3_model.hpp:410-436 initialize_rope. */
ei_status ei_build_rope_table(float* host_table, size_t max_positions, size_t head_dim, float theta);
/* ref: execution.hpp:106-109, execution.cu:374-386 store_kv<T>. */
ei_status ei_store_kv_bf16(const ei_context* ctx, ei_view2 source, ei_view2 capacity, size_t offset,
                           const size_t* device_offset);

/* ---- verify attention --------------------------------------------------------------------- */
/* Bytes of FP32 scratch for split-KV partials: q_rows query rows, kv_length cached tokens. */
size_t ei_attention_scratch_bytes(size_t q_rows, size_t query_heads, size_t head_dim, size_t kv_length);
/* ref: execution.hpp:118-122, execution.cu:402-417, kernels/flash_attn_prefill.cu:15-460
 * attention_prefill<T>(q [rows,heads,128], k/v [length,kv_heads,128], out, offset): causal attention
 * of `rows` query rows whose first row sits at absolute position `offset`. head_dim must be 128 and
 * rows * (heads / kv_heads) <= 128. KV is read once per KV head (shared by its query heads and rows),
 * split across blocks along the sequence and merged in FP32. */
ei_status ei_attention_prefill_bf16(const ei_context* ctx, ei_view3 q, ei_view3 k, ei_view3 v,
                                    ei_view3 out, size_t offset, void* scratch, size_t scratch_bytes);
/* Same computation for a captured graph: k/v describe the cache capacity and the offset of the first
 * query row is read from device memory at launch (the generalisation of the reference's graph-mode
 * device lengths, ref: execution.hpp:123-130, runtime/src/qwen3.cpp:356-367). Scratch must be sized
 * for kv_length = capacity. */
ei_status ei_attention_verify_bf16(const ei_context* ctx, ei_view3 q, ei_view3 k_capacity,
                                   ei_view3 v_capacity, ei_view3 out, const int32_t* device_offset,
                                   void* scratch, size_t scratch_bytes);

/* No counterpart in the reference. ei_attention_prefill_bf16 for callers that cannot supply scratch: a
 * plugin slot whose interface carries only the operator's tensors, a process that gave all device memory
 * to its own pool at start-up, a stateless hook with nowhere to keep a buffer between calls. The split
 * partials go to an array of EI_ATTENTION_STATIC_SCRATCH_BYTES that is part of the library image on every
 * device; the call never allocates or frees device memory. Same arguments, validation and results as
 * ei_attention_prefill_bf16 (bit-identical output). Limits and rules:
 *  - shapes whose split partials exceed the array are rejected with EI_INVALID_ARGUMENT before any write
 *    (the message states the bytes needed). The array holds 9 rows x 32 heads at any KV length; in
 *    general 64 * rows * heads * 528 bytes suffice;
 *  - the first call on each device resolves the array's address, with that device current; make that
 *    call before starting any stream capture;
 *  - every call on a device uses the same array, so two calls whose execution may overlap (different
 *    streams or threads) race; keep them on one stream or serialise them. Nothing in the array needs
 *    clearing between calls. */
#define EI_ATTENTION_STATIC_SCRATCH_BYTES (10u * 1024u * 1024u)
ei_status ei_attention_prefill_static_bf16(const ei_context* ctx, ei_view3 q, ei_view3 k, ei_view3 v,
                                           ei_view3 out, size_t offset);

/* ---- greedy sampling and acceptance -------------------------------------------------------------- */
/* Bytes of scratch for ei_sample_greedy_bf16. */
size_t ei_sample_scratch_bytes(size_t rows, size_t vocabulary);
/* ref: execution.hpp:146-151, execution.cu:463-498 sample<T> with top_k == 1 (greedy): per row the index
 * of the maximum logit, NaN treated as -inf, ties to the lowest index. One pass instead of a sort. */
ei_status ei_sample_greedy_bf16(const ei_context* ctx, ei_view2 logits, ei_view1 tokens, void* scratch,
                                size_t scratch_bytes);
/* Device-side result of one verify step. */
typedef struct ei_verify_result {
  int32_t emitted;      /* tokens emitted this step = KV rows retained (1..rows) */
  int32_t context;      /* context length after the commit */
  uint32_t tokens[16];  /* greedy target token of every row; the first `emitted` are the output */
} ei_verify_result;
/* ref: runtime/src/speculative_decoder.cpp:214-223 (host loop + KVCache::resize), done on the device:
 * inputs = [pending, d1..dk] (k = rows-1), targets = greedy token per row. Emits targets[0..m] where m is
 * the number of leading drafts with targets[i] == inputs[i+1]; adds m+1 to *context_length, writes
 * targets[m] to *pending and fills *result. Runs as one block; no host synchronisation. */
ei_status ei_verify_accept(const ei_context* ctx, const uint32_t* inputs, const uint32_t* targets,
                           size_t rows, int32_t* context_length, uint32_t* pending,
                           ei_verify_result* result);

/* ---- prepared model and session (runtime contract) -------------------------------------------------------- */
/* ref: runtime/include/models/qwen3_model.hpp:19-35 (Qwen3Config). */
typedef struct ei_model_config {
  uint64_t vocab_size, n_layers, n_heads, n_kv_heads, hidden_size, head_dim, intermediate_size,
      max_position_embeddings;
  uint32_t bos_token_id, eos_token_id;
  float rms_norm_eps, rope_theta;
  int32_t quant_type; /* 0 dense BF16, 1 AWQ int4 linears */
  int32_t group_size;
  int32_t qk_norm;
} ei_model_config;

/* One named tensor in the reference's weight-name schema (ref: qwen3_model.hpp:363-408):
 * token_embeddings.weight [V,H]; rms_out_w [H]; lm_head; rms_att_w{i}, rms_ffn_w{i} [H]; q_norm{i},
 * k_norm{i} [head_dim]; wq{i} wk{i} wv{i} wo{i} w_gate{i} w_up{i} w_down{i}; optional biases
 * layers.{i}.self_attn.{q,k,v,o}_proj.bias, layers.{i}.mlp.{gate,up,down}_proj.bias, lm_head.bias.
 * kind: 0 dense BF16, 1 AWQ qweight (int32), 2 AWQ scales (BF16), 3 AWQ zeros (int32).
 * A dense linear is given as the physical [out, in] matrix (each output's inputs contiguous).
 * `data` may be a host or a device pointer; it is copied into the model's own arena. */
typedef struct ei_named_tensor {
  const char* name;
  const void* data;
  uint64_t shape[2];
  int32_t rank;
  int32_t kind;
} ei_named_tensor;

typedef struct ei_model ei_model;
typedef struct ei_session ei_session;

/* ref: Qwen3Model<T> constructor (qwen3_model.hpp:283-305): copies every tensor into one private
 * device arena on the current device, resolves prepared linears and builds the RoPE table. Allocates. */
ei_status ei_model_create(const ei_model_config* config, const ei_named_tensor* tensors, size_t count,
                          ei_model** out);
void ei_model_destroy(ei_model* model);
ei_status ei_model_config_of(const ei_model* model, ei_model_config* out);
/* Bytes of prepared weights one verify step streams (layers + lm_head), the roofline numerator. */
size_t ei_model_weight_bytes(const ei_model* model);

/* ref: Qwen3Session<T>::create(model, capacity, graph) (runtime/src/qwen3.cpp:203-211): one stream,
 * workspace arena, device control block and a managed KV cache [layers, capacity, kv_heads*head_dim] x2.
 * `graph` != 0 replays each row count's step from a captured CUDA graph. Allocates. */
ei_status ei_session_create(ei_model* model, size_t capacity, int graph, ei_session** out);
void ei_session_destroy(ei_session* session);
/* ref: Qwen3Session<T>::prefill(host tokens) (qwen3.cpp:399-447): replaces the history. Returns a
 * borrowed device pointer to BF16 logits of the LAST row ([1, vocab]) in *last_logits, valid until the
 * session's next operation; all_logits (optional, device, BF16 [rows, vocab]) receives every row. */
ei_status ei_session_prefill(ei_session* session, const uint32_t* host_tokens, size_t rows,
                             const void** last_logits, void* all_logits);
/* ref: Qwen3Session<T>::decode(token) (qwen3.cpp:449-467): appends one token; logits [1, vocab]. */
ei_status ei_session_decode(ei_session* session, uint32_t token, const void** logits);
/* The verify step. ref: SpeculativeDecoder<T>::verify_greedy (runtime/src/speculative_decoder.cpp:200-224)
 * + verify_logits (:190-198) + Qwen3Session::prefill_eager. tokens = [pending, d1..dk], 1 <= rows <= 16.
 * One forward of `rows` tokens at the current context, greedy token per row, acceptance and KV
 * commit/rollback on the device, one host synchronisation at the end. *logits (optional) receives the
 * borrowed BF16 [rows, vocab] view. */
ei_status ei_session_verify(ei_session* session, const uint32_t* host_tokens, size_t rows,
                            ei_verify_result* result, const void** logits);
/* ---- several sessions in one forward --------------------------------------------------------------
 * No counterpart in the reference, whose sessions run one at a time. A batch is a fixed set of sessions of
 * one model (same device, same capacity, each listed once; at most 1024): ei_batch_verify stacks `rows`
 * (<= 16) tokens of each into one forward, so every weight is streamed once for all of them, while
 * attention, KV append, greedy acceptance and commit / rollback stay per session. host_tokens is
 * [sessions][rows] ([pending, d1..dk] of each session, in the order given to ei_batch_create), results is
 * [sessions]. Up to sessions * rows <= 16 stacked rows every session ends exactly as after its own
 * ei_session_verify with the same tokens (same bits). Above that, up to 2048 stacked rows and for models
 * whose projections the prompt GEMM takes, the forward runs on the tensor cores and one launch per kind of
 * kernel serves all sessions; results then agree with the single-session step within the rounding of another
 * summation order, and the sessions' logits buffers are not written. The step runs on the first session's
 * stream (and workspace, or the model's prompt workspace); the other sessions must not be in use from other
 * threads during the call. Destroy the batch before its sessions. */
typedef struct ei_batch ei_batch;
ei_status ei_batch_create(ei_session* const* sessions, size_t count, ei_batch** out);
void ei_batch_destroy(ei_batch* batch);
ei_status ei_batch_verify(ei_batch* batch, const uint32_t* host_tokens, size_t rows, ei_verify_result* results);

/* Asynchronous form for a device-resident loop: row 0 is the pending token kept on the device by the
 * previous step, row i >= 1 is device_drafts[context_length + i - draft_base]: device_drafts[j] is the
 * token proposed for absolute position draft_base + j, and row i of a step sits at position
 * context_length + i. Enqueues the step and returns without
 * synchronising; results accumulate in the session (ei_session_drain). */
ei_status ei_session_verify_enqueue(ei_session* session, const uint32_t* device_drafts, size_t draft_count,
                                    size_t draft_base, size_t rows);
/* Waits for enqueued steps; returns the last step's result and the total tokens emitted since the
 * previous drain. */
ei_status ei_session_drain(ei_session* session, ei_verify_result* last, uint64_t* emitted_total);
/* ref: KVCache<T>::resize (runtime/include/inference.hpp:41, runtime/src/inference.cpp:116-121) used for
 * EOS truncation (speculative_decoder.cpp:302-304): logical length only; must not exceed what is stored. */
ei_status ei_session_truncate(ei_session* session, size_t length);
/* Overrides the device-resident pending token (row 0 of the next enqueued step). */
ei_status ei_session_set_pending(ei_session* session, uint32_t token);
/* ref: Qwen3Session<T>::reset (qwen3.cpp:232-238). */
ei_status ei_session_reset(ei_session* session);
/* ref: context_size / context_capacity (qwen3.cpp:221-230), synchronize (:127-135), stream(). */
ei_status ei_session_context_size(const ei_session* session, size_t* out);
ei_status ei_session_context_capacity(const ei_session* session, size_t* out);
ei_status ei_session_synchronize(ei_session* session);
void* ei_session_stream(const ei_session* session);
/* Copies K and V rows [0, context) of one layer to the host as BF16 ([context, kv_heads*head_dim]). */
ei_status ei_session_read_kv(ei_session* session, size_t layer, void* host_k, void* host_v);
/* Restores a history: copies `rows` K and V rows (BF16, [rows, kv_heads*head_dim], host or device memory) of one
 * layer into cache rows [first, first + rows), on the session's stream, and waits. Together with
 * ei_session_adopt_history it moves a session's state (read with ei_session_read_kv) into another session of the
 * same model, or seeds a synthetic history for a benchmark. No counterpart in the reference (its KVCache is only
 * ever filled by its own forward passes, runtime/include/inference.hpp:71-106). */
ei_status ei_session_write_kv(ei_session* session, size_t layer, size_t first, size_t rows, const void* k,
                              const void* v);
/* Declares cache rows [0, length) valid and `pending` the next input token, as after a prefill of `length`
 * tokens whose greedy continuation is `pending`. length <= capacity, pending < vocabulary. */
ei_status ei_session_adopt_history(ei_session* session, size_t length, uint32_t pending);
/* Copies the first `rows` rows of the session's borrowed logits (BF16 [rows, vocab]) to the host: row 0 after
 * prefill / decode, rows 0..rows-1 after a verify step. */
ei_status ei_session_read_logits(ei_session* session, size_t rows, void* host_logits);
/* Kernels launched by this session's last step (the launches inside one captured graph). */
size_t ei_session_launches_per_step(const ei_session* session, size_t rows);

/* ---- draft + verify loop without host round trips ----------------------------------------------------
 * ref: SpeculativeDecoder<T>::generate_with_callback (runtime/src/speculative_decoder.cpp:227-306), whose round
 * is generate_draft_tokens (:176-187, one stream synchronisation per draft token) followed by verify_greedy
 * (:200-224, device-to-host copies and a host comparison). Here a round is enqueued as a whole: the draft
 * session decodes drafts_per_round + 1 tokens, each from the token its previous step left on the device, the
 * target session verifies [pending, d1..dk] in one forward, accepts and commits on the device, and the draft
 * session adopts the target's context length and pending token (both keep the pending input plus every
 * accepted one, :219-223). The host synchronises only in ei_speculative_drain. Greedy (top_k = 1) only, as the
 * reference. Both sessions must live on one device, share the vocabulary and must not be used directly while
 * the decoder drives them; destroy the decoder before its sessions. */
typedef struct ei_speculative ei_speculative;
ei_status ei_speculative_create(ei_session* target, ei_session* draft, size_t drafts_per_round,
                                ei_speculative** out);
void ei_speculative_destroy(ei_speculative* spec);
/* Starts a request: both sessions take the whole prompt; the target's greedy token after it is the first
 * generated token (*first_token, optional) and the pending token of both sessions. */
ei_status ei_speculative_prefill(ei_speculative* spec, const uint32_t* host_tokens, size_t rows,
                                 uint32_t* first_token);
/* Enqueues `rounds` rounds without synchronising. The host does not know the context length between drains and
 * bounds it by full acceptance: EI_LENGTH if that bound would pass the capacity (drain, then enqueue less). */
ei_status ei_speculative_enqueue(ei_speculative* spec, size_t rounds);
/* Waits for the enqueued rounds. *count = tokens generated since the prefill (the first token included);
 * host_tokens (optional, room for `capacity`) receives them from the first on; *last = the last verify step. */
ei_status ei_speculative_drain(ei_speculative* spec, uint32_t* host_tokens, size_t capacity, size_t* count,
                               ei_verify_result* last);
/* Keeps the first `generated` generated tokens (1 <= generated <= count): the last kept token becomes pending in
 * both sessions, the ones before it stay in both caches. ref: EOS truncation, speculative_decoder.cpp:302-304. */
ei_status ei_speculative_truncate(ei_speculative* spec, size_t generated);

/* Test hook (host-side fault injection, no GPU fault): the N-th next kernel launch of this session
 * fails with EI_RUNTIME before it is submitted (N = 0 disarms); `completion` != 0 makes the next stream
 * completion report failure after a real wait, which poisons the session.
 * ref: runtime/tests/qwen3_session_test.cpp:26-70 (link-time --wrap of cublasGemmEx / cudaStreamSynchronize). */
ei_status ei_session_inject_failure(ei_session* session, int nth_launch, int completion);

/* Test hook for the bounded device waits (no GPU fault, trap or endless loop is involved): the next
 * weight-streaming GEMM of this session runs outside any captured graph with a poll limit of `polls` and is
 * told to expect 16 bytes more than its first weight copy delivers, so the copy's barrier never completes, the
 * waits run out, the kernel returns and raises status bit 2. The step then reports EI_RUNTIME, the session's
 * own stream is drained and its history forgotten (prefill again); other sessions are untouched.
 * ref: the drain-or-poison rules of runtime/src/qwen3.cpp:127-161. No counterpart in the reference's API. */
ei_status ei_session_inject_wait_timeout(ei_session* session, uint32_t polls);
/* The same hook for the attention kernel: the first K / V tile copy of every block of this session's next
 * attention launch is told to expect 16 bytes more than it delivers. No counterpart in the reference's API. */
ei_status ei_session_inject_attention_wait_timeout(ei_session* session, uint32_t polls);

#ifdef __cplusplus
}
#endif
#endif /* EDGE_INFER_B200_H */
