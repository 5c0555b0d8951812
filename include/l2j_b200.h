/*
 * l2j_b200.h -- C ABI of libl2j_b200.so: llama2j's `--mode CUDA` token-decode path for NVIDIA B200.
 *
 * The library replaces what the reference's Java code reaches through JCuda for one token:
 * the device runtime (ContextCUDA.java), the run state (RunState.java), the device copies of the
 * weights (TransformerWeights.java) and the per-token forward (Run.transformerCUDA,
 * Run.java:315-519).  The Java host keeps its checkpoint reader, quant cache, tokenizer, sampler
 * and command line, and drives this ABI with java.lang.foreign downcalls.
 *
 * Paths in the comments are relative to the reference's src/main/java/com/lastbot/llama2j/.
 *
 * Conventions: every function returns 0 on success or a negative L2J_E_* code; the message of the
 * last failure of a context is available from l2j_last_error().  Nothing aborts or throws across
 * the ABI.  Host pointers only need to stay valid for the duration of the call.  There is no CPU
 * fallback: without a CUDA device l2j_create() fails.
 */
#ifndef L2J_B200_H
#define L2J_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported from the shared object (it is built with hidden default visibility). */
#if defined(__GNUC__)
#define L2J_API __attribute__((visibility("default")))
#else
#define L2J_API
#endif

#define L2J_OK 0
#define L2J_E_INVALID (-1)   /* bad argument, unsupported shape, wrong size */
#define L2J_E_CUDA (-2)      /* a CUDA runtime call failed */
#define L2J_E_STATE (-3)     /* call out of order (e.g. forward before finalize) */
#define L2J_E_DEVICE (-4)    /* a kernel reported a fault through the device status word */
#define L2J_E_NOMEM (-5)     /* device or host allocation failed */

/* Device status bits (l2j_stats.device_status): set by kernels, never by a trap. */
#define L2J_DS_WAIT_TIMEOUT 0x1  /* a bounded wait on a copy barrier ran out */
#define L2J_DS_BAD_POS 0x2       /* pos outside [0, seq_len) reached a kernel */
#define L2J_DS_BAD_TOKEN 0x4     /* token outside [0, vocab) reached a kernel */
#define L2J_DS_BAD_LINK 0x8      /* a stage of a layer split was told to read its neighbour but holds no pointer to it */

/* Quantisation group of the reference: Run.QUANT_GROUP_SIZE / QUANT_BITS, Run.java:27-28;
 * encoded group = 8-byte header (min, max as big-endian floats) + 256 bytes, Quant.java:35-37. */
#define L2J_QUANT_GROUP 256
#define L2J_QUANT_GROUP_BYTES 264

/* Config.java:6-13, plus the sign of vocab_size in the checkpoint header (Run.java:571-573). */
typedef struct l2j_config {
    int32_t dim;
    int32_t hidden_dim;
    int32_t n_layers;
    int32_t n_heads;
    int32_t n_kv_heads;
    int32_t vocab_size;        /* always positive here */
    int32_t seq_len;
    int32_t shared_classifier; /* 1: wcls is the embedding table (positive vocab in the file) */
} l2j_config;

/* Tensor ids, in checkpoint file order (TransformerWeights.java:50-122). */
enum l2j_tensor {
    L2J_T_TOKEN_EMBEDDING = 0, /* f32 (vocab, dim) */
    L2J_T_RMS_ATT = 1,         /* quant (layer, dim) */
    L2J_T_WQ = 2,              /* quant (layer, dim, dim) */
    L2J_T_WK = 3,              /* quant (layer, kv_dim, dim) */
    L2J_T_WV = 4,              /* quant (layer, kv_dim, dim) */
    L2J_T_WO = 5,              /* quant (layer, dim, dim) */
    L2J_T_RMS_FFN = 6,         /* quant (layer, dim) */
    L2J_T_W1 = 7,              /* quant (layer, hidden, dim) */
    L2J_T_W2 = 8,              /* quant (layer, dim, hidden) */
    L2J_T_W3 = 9,              /* quant (layer, hidden, dim) */
    L2J_T_RMS_FINAL = 10,      /* quant (dim) */
    L2J_T_WCLS = 11,           /* f32 (vocab, dim), only when not shared */
    L2J_T_COUNT = 12
};

/* l2j_create flags */
#define L2J_F_NO_GRAPH 0x1    /* launch kernels directly instead of replaying a CUDA graph */
#define L2J_F_NO_PDL 0x2      /* no programmatic dependent launch between consecutive kernels */
#define L2J_F_SIMPLE 0x4      /* plain direct-load matvec kernels (cross-check path, slower) */
#define L2J_F_STEP_KERNELS 0x8 /* one kernel per step of a layer (5 per layer) instead of one persistent kernel per token */
#define L2J_F_NO_TENSOR_PREFILL 0x40  /* l2j_prefill pushes the prompt through the decode step (what shapes the tensor-core path does not take get anyway) */
#define L2J_F_PERSISTENT 0x20  /* the persistent kernel wherever the shape allows it (default: only where it is the faster one) */
#define L2J_F_TP_SPLIT_CLASSIFIER 0x10 /* l2j_create_tp: split the classifier's rows over the ranks too (they exchange their best candidates) */

typedef struct l2j_ctx l2j_ctx;

typedef struct l2j_stats {
    int64_t forwards;          /* forwards launched since create/reset */
    int64_t kernels_per_forward;
    int64_t device_bytes;      /* device memory held by the context */
    int32_t device_status;     /* L2J_DS_* bits accumulated since create/reset */
    int32_t last_pos;
    int32_t last_token;        /* token chosen by the device argmax of the last forward */
    int32_t sm_count;
} l2j_stats;

/* ---- context ------------------------------------------------------------------------------- */

/* One context = one device and one contiguous layer range [first_layer, last_layer] of the model,
 * the unit LayerAllocation.java:67-95 assigns to a GPU.  A context that starts at layer 0 owns the
 * embedding gather (Run.java:362-363); one that ends at the last layer owns the final RMSNorm,
 * the classifier (Run.java:514-518) and the greedy pick (Sampler.java:46-57).
 * Replaces ContextCUDA's constructor (ContextCUDA.java:75-100) and RunState's device half
 * (RunState.java:107-166). */
L2J_API int l2j_create(const l2j_config *cfg, int device, int first_layer, int last_layer, uint32_t flags, l2j_ctx **out);

/* ContextCUDA.close(), ContextCUDA.java:311-323. */
L2J_API void l2j_destroy(l2j_ctx *ctx);

/* Message of the most recent failure on this context ("" if none).  ctx may be NULL for a
 * failure of l2j_create. */
L2J_API const char *l2j_last_error(const l2j_ctx *ctx);

/* ---- weights ------------------------------------------------------------------------------- */

/* Uploads (part of) a quantised tensor in the reference's group format, exactly the bytes of a
 * `.quant` cache file after its length field (BinFileWriter.java:20-34).  `float_offset` is the
 * index of the part's first element in the whole tensor and must be a multiple of 256; `n_floats`
 * is the number of elements in the part; `bytes` must equal ceil(n_floats/256)*264.  Parts outside
 * the context's layer range are ignored, parts that overlap it are clipped.  Replaces
 * ContextCUDA.allocateQuantAndCopyToDevice (ContextCUDA.java:138-158) and the SPLIT_TO_LAYERS /
 * LAST_DEVICE_ONLY policies (TransformerWeights.java:238-350).  Thread-safe per context. */
L2J_API int l2j_upload_quant(l2j_ctx *ctx, int tensor, int64_t float_offset, const void *groups, int64_t bytes,
                     int64_t n_floats);

/* Uploads (part of) an FP32 tensor: the embedding table or the unshared classifier
 * (TransformerWeights.java:119-135). */
L2J_API int l2j_upload_f32(l2j_ctx *ctx, int tensor, int64_t float_offset, const float *data, int64_t n_floats);

/* Checks that every tensor the layer range needs has arrived, builds the derived tables and
 * captures the per-token graph.  Must follow the uploads and precede the first forward. */
L2J_API int l2j_finalize(l2j_ctx *ctx);

/* ---- per-token forward --------------------------------------------------------------------- */

/* One decode step: Run.transformerCUDA(token, pos, ...) (Run.java:315-519) followed by the
 * logits read-back of the run loop (Run.java:628-632).  For a context that holds the whole model.
 * `logits` (vocab floats) and `argmax` may each be NULL.  Blocks until the results are on the host. */
L2J_API int l2j_forward(l2j_ctx *ctx, int token, int pos, float *logits, int *argmax);

/* The same step for one stage of a layer split.  A first stage takes `token`; later stages take
 * the activation vector x (dim floats, host memory) that the previous stage returned, the hand-off
 * of Run.java:368-413.  A stage that is not the last writes its x to `x_out`; the last stage fills
 * `logits` / `argmax`.  Unused pointers may be NULL. */
L2J_API int l2j_forward_stage(l2j_ctx *ctx, int token, int pos, const float *x_in, float *x_out, float *logits, int *argmax);

/* Device addresses of the stage's activation vector x (dim floats) and of its logits, for callers
 * that move them with their own device-to-device transport. */
/* Batched prompt processing (no counterpart in the reference, whose run loop pushes every prompt token through
 * the decode step, Run.java:623-637): positions pos0 .. pos0 + n - 1 with the input tokens given (tokens[i] is
 * the token fed at position pos0 + i, i.e. BOS and then the prompt, Run.java:614,635-637), 64 positions per
 * sweep over the weights, dot products on the tensor cores (u8 weights x s8 limbs of the 24-bit fixed-point
 * activations, exact integer sums, group (min, scale) applied in FP32 as in the decode kernels).  Leaves the K/V
 * cache as the decode steps would leave it to FP32 rounding of the row sums (prompt positions are not bitwise
 * those of the decode kernels); produces no logits: continue with l2j_forward(token, pos0 + n).  Needs a
 * context that holds every layer.  Shapes the tensor-core path does not take (rows that are not whole
 * quantisation groups, head sizes other than 64 and 128) go through the decode step, as with
 * L2J_F_NO_TENSOR_PREFILL; l2j_prefill_launches tells which ran (kernels launched by the batched path so far). */
L2J_API int l2j_prefill(l2j_ctx *ctx, const int32_t *tokens, int n, int pos0);
L2J_API uint64_t l2j_prefill_launches(l2j_ctx *ctx);

/* Concurrent sequences on one sweep over the weights (the reference's roadmap item "parallel processing of
 * multiple queries", README.md:347,355-360; it has no such path).  l2j_batch_create gives the context K/V caches
 * for n_seq independent sequences of seq_len positions (beside the cache of the single sequence, which
 * l2j_forward keeps using).  l2j_batch_forward runs ONE decode step for up to 64 entries (sequence seq[i] is fed
 * tokens[i] at position pos[i]): every weight byte is read once for all of them, dot products on the tensor
 * cores as in l2j_prefill, attention per entry over its own sequence's cache, FP32 classifier for all entries.
 * logits (n x vocab floats) and argmax (n ints, first maximum) may be NULL.  A sequence may appear with several
 * positions in one call (a prompt in slices of 64): their K/V rows are written before any attention runs.
 * Per entry the arithmetic is the decode step's with the row sums in another order (agreement to rounding, not
 * bit for bit, with l2j_forward). */
L2J_API int l2j_batch_create(l2j_ctx *ctx, int n_seq, int seq_len);
L2J_API int l2j_batch_forward(l2j_ctx *ctx, int n, const int32_t *seq, const int32_t *pos, const int32_t *tokens, float *logits,
                              int32_t *argmax);

/* Token selection on the device for --temp > 0 (Run.java:643-665 with Sampler.java:20-44,76-120): the logits
 * of the last forward are divided by the temperature, turned into probabilities in place exactly as the
 * reference does it (exp in double, one sequential float sum) and sampled plainly (topp > 0.999) or from the
 * nucleus, with java.util.Random's 48-bit generator seeded like `new Sampler(seed, vocab)`: from the same
 * logits the device chooses the token the Java Sampler chooses, and only its id crosses PCIe (call
 * l2j_forward with logits == NULL).  The ProbIndex array the reference keeps across calls (and sorts whole,
 * stale entries included) is kept across calls here too.  temperature == 0 returns the arg-max
 * (Sampler.argmax).  Vocabularies of at most 39,000 tokens (the probabilities live in shared memory). */
L2J_API int l2j_sampler_seed(l2j_ctx *ctx, int64_t seed);
L2J_API int l2j_sample(l2j_ctx *ctx, float temperature, float topp, int *token);

L2J_API int l2j_device_buffers(l2j_ctx *ctx, void **x_dev, void **logits_dev);

/* The stage step without host copies: enqueues the kernels on the context's stream and returns.
 * x must already be in the device buffer (or token given for a first stage). */
L2J_API int l2j_forward_stage_async(l2j_ctx *ctx, int token, int pos);

/* Waits for the context's stream and returns L2J_E_DEVICE if a kernel raised a status bit. */
L2J_API int l2j_sync(l2j_ctx *ctx);

/* The run loop of Run.java:609-685 with greedy selection, kept on the device: position 0 is fed
 * BOS (token 1), positions 1..n_prompt are fed the prompt, later positions the previous argmax.
 * `out_tokens[p]` receives the token chosen after position p (the forced prompt token while the
 * prompt lasts), for p in [0, steps).  No host round trip between tokens; the early stop on a
 * sampled BOS (Run.java:670-672) is left to the caller, who truncates. */
L2J_API int l2j_generate_greedy(l2j_ctx *ctx, const int32_t *prompt, int n_prompt, int steps, int32_t *out_tokens);

/* ---- layer split over several devices, one host thread (Run.java:368-413) ------------------- */

/* Connects contexts that tile the layers in order (stage 0 from layer 0, the last stage with the
 * classifier), one per device as `--gpuMem a,b,...` creates them (LayerAllocation.java:54-95,
 * Context.java:16-23).  Afterwards a stage reads the activation vector x straight from the previous
 * stage's device memory over the peer link, where the reference copies it through a host array
 * with two blocking synchronisations (ContextCUDA.java:269-280).  Needs peer access between the
 * devices of neighbouring stages; returns L2J_E_STATE without it (l2j_forward_stage still works). */
L2J_API int l2j_pipeline_link(l2j_ctx *const *stages, int n_stages);

/* One decode step over linked stages: the loop over devices of Run.transformerCUDA.  Each stage's
 * stream waits for the stage in front through an event; the host blocks only at the end. */
L2J_API int l2j_pipeline_forward(l2j_ctx *const *stages, int n_stages, int token, int pos, float *logits, int *argmax);

/* l2j_generate_greedy over linked stages: the chosen token stays on the last stage's device and the
 * first stage reads it from there.  l2j_last_generate_us(stages[0]) gives the device time. */
L2J_API int l2j_pipeline_generate_greedy(l2j_ctx *const *stages, int n_stages, const int32_t *prompt, int n_prompt, int steps,
                                         int32_t *out_tokens);

/* ---- tensor-parallel group, one host thread (no counterpart in the reference) ---------------- */

/* A context that holds every layer but works on rank `tp_rank`'s block of rows of each matrix
 * (whole heads for Wq/Wk/Wv and the attention, hidden_dim / tp_size rows of W1/W3, dim / tp_size
 * rows of Wo/W2; the classifier is computed by every rank unless L2J_F_TP_SPLIT_CLASSIFIER is given, which
 * splits its rows too and lets the ranks exchange their best candidates).
 * Each rank sends its results to every rank over the peer links as (value, sequence number) pairs;
 * every output element is computed by one rank in the order of the single device's per-step kernels, so
 * logits and tokens are bitwise those of one device created with L2J_F_STEP_KERNELS.  Weights are uploaded to every rank with the usual calls.  n_heads,
 * n_kv_heads and hidden_dim must divide by tp_size (at most 8).  The reference has no such mode
 * (its multi-GPU mode is the layer split above). */
L2J_API int l2j_create_tp(const l2j_config *cfg, int device, int tp_rank, int tp_size, uint32_t flags, l2j_ctx **ctx);

/* Connects the finalized contexts of ranks 0..n-1, each on a device of its own with peer access to
 * the others (kernels of different ranks wait for each other, with a time limit: they must not
 * share a device). */
L2J_API int l2j_tp_link(l2j_ctx *const *ranks, int n_ranks);

/* l2j_forward / l2j_generate_greedy over a linked group; results are read from rank 0. */
L2J_API int l2j_tp_forward(l2j_ctx *const *ranks, int n_ranks, int token, int pos, float *logits, int *argmax);
L2J_API int l2j_tp_generate_greedy(l2j_ctx *const *ranks, int n_ranks, const int32_t *prompt, int n_prompt, int steps,
                                   int32_t *out_tokens);

/* Clears the KV cache position bookkeeping, the statistics and the device status word (a new sequence).
 * The status word is sticky: once a kernel has raised a bit, every later forward of the context returns
 * L2J_E_DEVICE (and, after L2J_DS_WAIT_TIMEOUT, its waits give up after 2 us, so its results are not valid)
 * until l2j_reset.  The hand-over counters of a context only agree with those of its partners (the ranks of
 * a tensor-parallel group, the stages of a linked layer split) while all of them have run the same number of
 * forwards: after a failure reset every member, l2j_tp_reset / l2j_pipeline_reset do that. */
L2J_API int l2j_reset(l2j_ctx *ctx);
L2J_API int l2j_tp_reset(l2j_ctx *const *ranks, int n_ranks);
L2J_API int l2j_pipeline_reset(l2j_ctx *const *stages, int n_stages);

/* Bound of every device-side wait of the context's kernels (copy barriers, hand-over counters between
 * kernels and between the blocks of the persistent kernel, the pair polls of a tensor-parallel group), in
 * microseconds; 50000 unless set.  A wait that runs out raises L2J_DS_WAIT_TIMEOUT and the kernel carries on,
 * so the GPU never hangs on a lost partner (the reference's only failure handling is the exception of
 * ContextCUDA.java:296-304).  Part of the captured launches: call before l2j_finalize. */
L2J_API int l2j_set_wait_limit_us(l2j_ctx *ctx, int limit_us);

/* Failure injection for tests, on the host: makes the context's next forward wait for hand-overs that never
 * come (its forward counter is advanced as if a partner had run a forward that this context missed).  The
 * forward then ends by its wait limit with L2J_E_DEVICE / L2J_DS_WAIT_TIMEOUT; l2j_reset makes the context
 * usable again.  Nothing faults: every wait gives up and the kernels return. */
L2J_API int l2j_debug_desync(l2j_ctx *ctx);

L2J_API int l2j_get_stats(l2j_ctx *ctx, l2j_stats *out);

/* How the per-token work is issued: bit 0 CUDA graph replay, bit 1 programmatic dependent launch
 * between kernels, bit 2 the bulk-copy ring kernels (else the plain kernels), bit 3 all layers of a token in
 * one persistent launch (else five launches per layer); bits 8 and up hold the number of blocks a ring
 * kernel is launched with.  The reference issues
 * every kernel with its own cuLaunchKernel (kernel/MatMul.java:338-354). */
L2J_API int l2j_launch_mode(l2j_ctx *ctx);

/* Reads a run-state buffer after a forward, the device half of RunState.java:38-50, for
 * stage-by-stage comparison in the spirit of the reference's TEST mode (Run.java:186-303):
 * which = 0 x, 1 attention output xb, 2 q, 3 hb, 4 logits (layer/pos ignored);
 * 5 K row, 6 V row of (layer, pos) in the reference's (kv_dim) order, n must be kv_dim. */
L2J_API int l2j_read_buffer(l2j_ctx *ctx, int which, int layer, int pos, float *out, int n);

/* Restores part of the KV cache from the host: rows [pos0, pos0 + n_pos) of `layer`, given as the
 * reference holds them, (position, kv_dim) floats (RunState.java:141-151, Run.java:438-444); the
 * library re-lays them out into its own (kv_head, position, head) order.  With it a harness can put a
 * long prompt's cache back instead of pushing the prompt through the decode path again, and a test can
 * give the device and the CPU checker the same cache.  Blocks until the rows are on the device. */
L2J_API int l2j_kv_write(l2j_ctx *ctx, int layer, int pos0, int n_pos, const float *k_rows, const float *v_rows);

/* Average device time in microseconds of the last l2j_generate_greedy call per forward, measured
 * with CUDA events on the context's stream. */
L2J_API int l2j_last_generate_us(l2j_ctx *ctx, double *total_us);

/* Measurement aid (the reference only prints tok/s, Run.java:703-706): average device time in
 * microseconds of one launch of each kernel of a layer at position `pos`, timed with CUDA events on
 * the context's stream over `reps` sweeps through all layers (so consecutive launches never re-read
 * the same weights).  us[0..5] = QKV+RoPE, attention, Wo+residual, W1/W3+SwiGLU, W2+residual,
 * classifier+argmax.  Leaves the sequence state undefined: call l2j_reset afterwards. */
L2J_API int l2j_time_kernels(l2j_ctx *ctx, int pos, int reps, double *us);

/* The same for the persistent kernel that runs all layers of a token in one launch (contexts created
 * without L2J_F_STEP_KERNELS whose matrices have rows of whole quantisation groups): average device time
 * of one launch at position `pos`, CUDA events on the context's stream around the launch alone, each
 * launch after an embedding gather of its own.  Leaves the sequence state undefined: call l2j_reset. */
L2J_API int l2j_time_layers_kernel(l2j_ctx *ctx, int pos, int reps, double *us_per_launch);

/* Measurement aid (no counterpart in the reference): the in-kernel timeline of one launch of a ring
 * kernel (kind 0 QKV, 2 Wo, 3 W1/W3, 4 W2, 5 classifier; same numbering as l2j_time_kernels).
 * out receives 16 values per block for up to max_blocks blocks: SM cycle counter at 0 block entry,
 * 1 first bulk copy issued, 2 last bulk copy issued, 3 consumer prologue done, 4 first stage landed,
 * 5 consumers done, 6 epilogue warp done; 7 / 8 = global timer in ns at block entry / epilogue done;
 * 9-15 finer marks of the block set-up.
 * Leaves the sequence state undefined: call l2j_reset afterwards. */
L2J_API int l2j_trace_kernel(l2j_ctx *ctx, int kind, int layer, int pos, uint64_t *out, int max_blocks);

/* The same timelines for every ring-kernel launch of the last forward, in launch order (per layer
 * QKV, Wo, W1/W3, W2, then the classifier), 16 values per block and two blocks per SM.  Only
 * recorded when the context was created with L2J_TRACE set in the environment. */
L2J_API int l2j_read_trace(l2j_ctx *ctx, uint64_t *out, int64_t max_values);

/* ---- load-time helpers on the device ------------------------------------------------------- */

/* Quant.encode (Quant.java:156-193) on the device, bit-exact: `in` host floats -> `out` host
 * bytes (ceil(n/256)*264).  `device` selects the GPU. */
L2J_API int l2j_quant_encode(int device, const float *in, int64_t n_floats, void *out);

/* Synthetic checkpoint tensors (no counterpart in the reference, which loads real checkpoints):
 * element i of stream `stream` is a counter-based N(0,1) draw times `scale`.  The f32 form writes
 * host floats; the quant form generates and encodes on the device and writes the group format. */
L2J_API int l2j_synth_f32(int device, uint64_t seed, uint32_t stream, int64_t start, int64_t n_floats, float scale,
                  float *out);
L2J_API int l2j_synth_quant(int device, uint64_t seed, uint32_t stream, int64_t n_floats, float scale, void *out);

/* ---- single-kernel entry points (TEST-mode counterparts, Run.java:186-303) ------------------ */

/* xout = W x with fused dequantisation: MatMul.callI8 (kernel/MatMul.java:314-358).
 * `groups` is the whole tensor in group format on the host, `weight_index` the element index of
 * W's first entry (l * d * n in the reference's call sites), n the row length, d the row count. */
L2J_API int l2j_k_matvec_i8(int device, uint32_t flags, const void *groups, int64_t tensor_floats, int64_t weight_index,
                    int n, int d, const float *x, float *xout);

/* xout = W x, FP32 weights: MatMul.callFP32 (kernel/MatMul.java:289-312). */
L2J_API int l2j_k_matvec_f32(int device, uint32_t flags, const float *w, int n, int d, const float *x, float *xout,
                     int *argmax);

/* out = deq(w) * (rsqrt(mean(x^2) + 1e-5) * x): RootMeanSquare.call + WeightNormalizeAndScale.callI8
 * (kernel/RootMeanSquare.java:57-118, kernel/WeightNormalizeAndScale.java:141-189). */
L2J_API int l2j_k_rmsnorm(int device, const void *groups, int64_t tensor_floats, int64_t weight_index, int n,
                  const float *x, float *out);

/* ApplyRope.call (kernel/ApplyRope.java:114-142): rotates q (dim) and k (kv_dim) in place. */
L2J_API int l2j_k_rope(int device, float *q, float *k, int pos, int dim, int kv_dim, int head_size);

/* AttentionLoop + ExpSumNormalize + AccumWeightedValue for every head (Run.java:450-478).
 * key/value caches are in the reference's layout (seq, kv_dim) for one layer; positions 0..pos
 * are read.  out receives n_heads * head_size floats. */
L2J_API int l2j_k_attention(int device, const float *q, const float *key_cache, const float *value_cache, int pos,
                    int n_heads, int n_kv_heads, int head_size, int seq_len, float *out);

/* Silu.call (kernel/Silu.java:97-135): hb = hb * sigmoid(hb) * hb2. */
L2J_API int l2j_k_swiglu(int device, float *hb, const float *hb2, int n);

/* No counterpart in the reference.  The attention step for hosts that must not allocate device memory
 * while they run (a process whose memory pool belongs to another allocator, a latency-bound loop that
 * cannot afford cudaMalloc's implicit synchronisation): the same kernel as l2j_k_attention, but all
 * pointers are device pointers supplied by the caller, the caches are in the library's own layout
 * (kv_head, position, head_size) with row stride seq_len, and the split-merge scratch is a fixed
 * ~2.1 MB array inside the library that every GPU loading it holds until exit.  Limits: at most 128
 * heads of at most 128 floats; larger problems are rejected with L2J_E_INVALID.  The call only enqueues
 * work on `stream` (a cudaStream_t, NULL for the default stream) and does not synchronise; it calls no
 * cudaMalloc / cudaFree.  The first call on a device looks up the scratch array's device address, so
 * make it before any stream capture.  All calls share the one array: two calls whose kernels overlap
 * on the GPU race on it, keep them on one stream or order them yourself.  `stream` must be a stream of
 * `device` (or 0); the call makes `device` current for the duration and puts the caller's device back. */
L2J_API int l2j_k_attention_noalloc(int device, const float *q_dev, const float *k_cache_dev, const float *v_cache_dev,
                                    int pos, int n_heads, int n_kv_heads, int head_size, int seq_len, float *out_dev,
                                    void *stream);

/* Message of the calling thread's most recent l2j_k_attention_noalloc failure ("" if none). */
L2J_API const char *l2j_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif

#endif /* L2J_B200_H */
