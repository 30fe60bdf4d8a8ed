/*
 * efm_b200.h — C ABI of the B200 (sm_100a) device backend for EdgeFM's single-request
 * generate() path.
 *
 * The reference engine (windog-labs/edge-fm-x) has no FFI boundary on this path: its
 * StandardEngine calls C++ Model/Layer/Operator objects directly.  This header is the
 * boundary a reference-side engine binds instead; each entry point names the reference
 * interface it replaces (paths relative to the reference tree).  Style follows the one
 * thin backend boundary the reference does have, IRuntimeBackend
 * (src/backends/runtime_backend.h:56-75): integer status + last_error().
 *
 * Rules: plain C types only; every call returns efm_status (0 = ok) and records a message
 * retrievable with efm_b200_last_error(); no exceptions cross the boundary; a context is
 * owned by one host thread at a time; all device work runs on the context's own stream.
 * There is no CPU fallback: every entry point fails with EFM_ERR_CUDA when no sm_100 device
 * is usable.
 */
#ifndef EFM_B200_H_
#define EFM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define EFM_API
#else
#define EFM_API __attribute__((visibility("default")))
#endif

typedef int32_t efm_status;
enum {
    EFM_OK = 0,
    EFM_ERR_INVALID_ARGUMENT = 1,
    EFM_ERR_CUDA = 2,
    EFM_ERR_OUT_OF_MEMORY = 3,
    EFM_ERR_STATE = 4,         /* call order violated (e.g. decode before prefill) */
    EFM_ERR_UNSUPPORTED = 5,   /* shape / dtype outside what the kernels are built for */
    EFM_ERR_DEVICE_WAIT = 6    /* a bounded device-side wait gave up; context still usable */
};

/* element types, numbered like edge_fm::DType (include/edge-fm/core.h:17-25) */
enum { EFM_F32 = 0, EFM_F16 = 1, EFM_BF16 = 2, EFM_I32 = 3, EFM_I64 = 4, EFM_U8 = 5, EFM_I8 = 6 };
/* where a caller buffer lives */
enum { EFM_MEM_HOST = 0, EFM_MEM_DEVICE = 1 };

/* Model geometry: the fields the reference reads from the HF config.json
 * (src/models/model.cpp:56-71, src/models/qwen2_5/qwen2_5.cpp:89-93,172-200). */
typedef struct efm_model_desc {
    int32_t struct_size;          /* = sizeof(efm_model_desc) */
    int32_t num_layers;
    int32_t hidden;
    int32_t q_heads;
    int32_t kv_heads;
    int32_t head_dim;             /* 64 or 128 */
    int32_t intermediate;         /* multiple of 64 */
    int32_t vocab;                /* even */
    float rms_eps;
    float rope_theta;
    int32_t tied_lm_head;         /* 1: lm_head reads model.embed_tokens.weight */
    int32_t use_mrope;            /* 1: positions come as [3,S] rows (Qwen2.5-VL) */
    int32_t mrope_section[3];     /* rotary pairs per row, e.g. {16,24,24} */
    int32_t max_prefill_tokens;   /* activation rows; longer prefills are chunked */
    int32_t max_response_tokens;  /* capacity of the device-side response buffer */
} efm_model_desc;

/* sampling.{temperature,top_p,top_k,seed} of the engine JSON (src/layers/sampler.cu:121-133).
 * temperature < 1e-6 -> greedy (ties -> lowest id).  top_k is accepted and ignored, as in
 * the reference. */
typedef struct efm_sampling {
    float temperature;
    float top_p;
    int32_t top_k;
    uint32_t reserved;
    uint64_t seed;
} efm_sampling;

typedef struct efm_b200_ctx efm_b200_ctx;

/* ---- lifetime -------------------------------------------------------------------------- */
/* Replaces Model::create + Qwen2_5 ctor (src/models/model.cpp:74-85, qwen2_5.cpp:84-246).
 * tp_rank/tp_size: tensor-parallel coordinates (1 rank = whole model). */
EFM_API efm_status efm_b200_create(const efm_model_desc* desc, int32_t device_id, int32_t tp_rank,
                                   int32_t tp_size, efm_b200_ctx** out);
EFM_API efm_status efm_b200_destroy(efm_b200_ctx* ctx);
/* Message of the last failing call on this context (ctx may be NULL: last create failure). */
EFM_API const char* efm_b200_last_error(const efm_b200_ctx* ctx);
EFM_API const char* efm_b200_version(void);

/* ---- tensor parallel (no counterpart in the reference, which is single-GPU) ------------------ */
/* One context per rank / GPU.  Rank 0 draws a 128-byte communicator id, the host code carries it to
 * the other ranks (any transport), every rank then calls tp_init before its first prefill.  Heads
 * and MLP columns are sharded inside set_weight (callers always pass whole tensors); row-parallel
 * outputs are summed with an NCCL all-reduce on the context stream (captured in the decode graph). */
EFM_API efm_status efm_b200_tp_unique_id(void* out128);
EFM_API efm_status efm_b200_tp_init(efm_b200_ctx* ctx, const void* id128);

/* Optional: fuse the two all-reduces per layer of the DECODE step into the GEMV kernels.  Every rank exports a
 * 64-byte handle of its exchange buffer (CUDA IPC), the host gathers the tp_size handles in rank order and
 * hands the whole array to every rank.  After import — and a host-side barrier across the ranks, so that
 * nobody decodes before everybody imported — each row-parallel GEMV stores its fp32 partial straight into
 * every peer's buffer over NVLink as 8-byte {value, exchange count} words; the next kernel's prologue re-reads
 * (bounded, EFM_ERR_DEVICE_WAIT on expiry) until every word carries the current count and adds the partials in
 * rank order.  Without these two calls
 * the decode step uses ncclAllReduce.  Prefill exchanges its [S, hidden] partials through the same peer buffers
 * (copy + published count + ordered add) once they are imported; the logits all-gather stays on NCCL. */
EFM_API efm_status efm_b200_tp_peer_export(efm_b200_ctx* ctx, void* handle64);
EFM_API efm_status efm_b200_tp_peer_import(efm_b200_ctx* ctx, const void* handles, int32_t n_handles);

/* Failure detection (the reference, being single-GPU, only surfaces CUDA errors at the final stream sync:
 * src/utils/device/cuda_utils.h:27-33).  Two limits, 0 keeps the current value:
 *   device_wait_us  longest a kernel waits, in total, for its peers' words / flags before it raises the device status
 *                   (EFM_ERR_DEVICE_WAIT from read_tokens; later kernels see the status and do not wait again, and
 *                   decode_steps stops queueing).  Default 2 s, or $EFM_B200_PEER_WAIT_MS.  Re-captures decode graphs.
 *   host_timeout_s  limit of every synchronising call (read_tokens, read_logits, synchronize) on a tensor-parallel
 *                   context; while it waits the call polls ncclCommGetAsyncError.  On an NCCL error (EFM_ERR_CUDA) or on
 *                   expiry (EFM_ERR_DEVICE_WAIT) the communicator is aborted and the context is only good for destroy.
 *                   Default 300 s, or $EFM_B200_TP_TIMEOUT_S. */
EFM_API efm_status efm_b200_tp_set_wait_limit(efm_b200_ctx* ctx, int64_t device_wait_us, double host_timeout_s);
/* The host-side wait itself, for engines that wait on their own streams by the same rule: polls ready(arg) (non-zero =
 * done) about once per millisecond and the communicator's asynchronous error state in between.  nccl_comm may be NULL
 * (timeout only).  EFM_OK / EFM_ERR_CUDA (NCCL error; communicator aborted) / EFM_ERR_DEVICE_WAIT (timeout; aborted).
 * Needs no GPU by itself. */
EFM_API efm_status efm_b200_tp_host_wait(void* nccl_comm, int (*ready)(void*), void* arg, double timeout_s);

/* ---- weights --------------------------------------------------------------------------- */
/* Replaces WeightLoader::load_weights_from_file + per-layer load_weights
 * (src/utils/device/weight_loader.cpp:80-171, src/layers/linear.cu:1691-1717,1926-1943).
 * hf_name: e.g. "model.layers.3.self_attn.q_proj.weight"; data is row-major [out,in] bf16.
 * Unknown names are ignored (returns EFM_OK), like the reference's name filter.  A device-resident
 * source (EFM_MEM_DEVICE) is read on the context's own stream: whatever produced it must have finished. */
EFM_API efm_status efm_b200_set_weight(efm_b200_ctx* ctx, const char* hf_name, const void* data,
                                       const int64_t* shape, int32_t ndim, int32_t dtype, int32_t mem_kind);
/* Group-wise INT4 (W4A16) weights for the DECODE pass only, from a second checkpoint (the reference's
 * decode_model_path, src/engine/engine_factory.cpp:64-72; weight contract src/layers/linear.cu:536-565):
 *   "<linear>.qweight"          int8 [out_features / 2, in_features]: byte [r][k] carries rows 2r (low nibble) and
 *                               2r + 1 (high nibble) of column k as q + 8, q in [-8, 7];
 *   "<linear>.scaling_factors"  fp16 or bf16 [in_features / 128, out_features];  w[n][k] = q[n][k] * scale[k / 128][n]
 * for <linear> = model.layers.N.{self_attn.{q,k,v,o}_proj, mlp.{gate,up,down}_proj} (all layers or none) and, optionally,
 * lm_head.  Prefill keeps the bf16 weights of efm_b200_set_weight; biases, norms and the embedding table are shared.
 * finalize_weights re-packs the tensors into the decode kernel's layout.  The nibble order inside the reference's
 * qweight is produced by a packer that is not part of its tree (TensorRT-Edge-LLM); the plain order above is this
 * library's own, so checkpoints packed for the reference's kernels have to be re-packed.  Other tensor names are
 * ignored; tensor-parallel contexts refuse INT4 weights, and in_features must be a multiple of 128 (EFM_ERR_UNSUPPORTED). */
EFM_API efm_status efm_b200_set_decode_weight(efm_b200_ctx* ctx, const char* hf_name, const void* data,
                                              const int64_t* shape, int32_t ndim, int32_t dtype, int32_t mem_kind);
/* Checks that every tensor arrived; after this call weights are immutable. */
EFM_API efm_status efm_b200_finalize_weights(efm_b200_ctx* ctx);

/* ---- KV slots -------------------------------------------------------------------------- */
/* Replaces KVManager slot allocation (src/engine/tasks/token_generation/kv_manager.cpp:45-201):
 * per layer one buffer [K: max_tokens x kv_heads x head_dim | V: same], bf16. */
EFM_API efm_status efm_b200_alloc_kv_slot(efm_b200_ctx* ctx, int32_t slot, int32_t max_tokens);
/* Device address of layer's K block for the slot (V block follows at +max_tokens*kv*D elements);
 * KVManager::get_read_kvcache (kv_manager.cpp:203-230). */
EFM_API efm_status efm_b200_kv_layer_ptr(efm_b200_ctx* ctx, int32_t slot, int32_t layer, void** k_base,
                                         int32_t* max_tokens);

/* ---- generate path --------------------------------------------------------------------- */
/* Replaces SamplerLayer configuration (src/layers/sampler.cu:121-133). */
EFM_API efm_status efm_b200_set_sampling(efm_b200_ctx* ctx, const efm_sampling* s);

/* Replaces prepare_prefill_tensors + Qwen2_5::prefill + run_sampler
 * (standard_engine.cpp:1200-1477,925-971; qwen2_5.cpp:534-930).
 * Runs the model over n_tokens ids (host int32) whose KV lands at cache rows
 * [kv_offset, kv_offset+n_tokens); rows [0,kv_offset) must already be resident (fixed prefix).
 * embeds (bf16 [n_embeds, hidden], host or device per embeds_mem) replace ids in
 * [embed_token_id, embed_token_id+n_embeds) (src/layers/embed_head.cu:93-116); pass NULL/0/-1
 * for none.  pos_ids3: host int32 [3, n_tokens] for M-RoPE models, else NULL.
 * When sample != 0 the last row's logits are sampled (RNG counter 0) into the device token
 * slot and response position 0. */
EFM_API efm_status efm_b200_prefill(efm_b200_ctx* ctx, int32_t slot, const int32_t* token_ids,
                                    int32_t n_tokens, int32_t kv_offset, const void* embeds,
                                    int32_t n_embeds, int32_t embed_token_id, int32_t embeds_mem,
                                    const int32_t* pos_ids3, int32_t sample);

/* Prefill CUDA graphs for short prompts (try_run_prefill_cuda_graph, standard_engine.cpp:568-770: one graph per
 * request id and sequence length, token ids refreshed before each replay).  When enabled, a prefill that fits one chunk
 * (n_tokens <= max_prefill_tokens) is launched kernel by kernel the first time its shape (slot, n_tokens, kv_offset,
 * injected-embedding count / id, sample flag, attention kind) is seen, captured the second time and replayed afterwards;
 * ids, positions, embeddings and the state words are copied into stable device buffers before each launch.  At most 8
 * shapes are kept (least recently used out).  Off by default; the engine turns it on with runtime.use_cuda_graph. */
EFM_API efm_status efm_b200_set_prefill_graph(efm_b200_ctx* ctx, int32_t enable);
/* Graphs currently held and replays so far (either pointer may be NULL). */
EFM_API efm_status efm_b200_prefill_graph_stats(efm_b200_ctx* ctx, int32_t* captured, int64_t* replays);

/* Which attention kernel efm_b200_prefill uses: 0 = bf16 flash attention (default), 1 = the INT8 scheme of
 * efm_b200_op_sage_prefill_attention.  Allocates the INT8 scratch for the largest KV slot allocated so far;
 * call it after efm_b200_alloc_kv_slot.  Decode is unaffected. */
EFM_API efm_status efm_b200_set_prefill_attention(efm_b200_ctx* ctx, int32_t kind);

/* Replaces prepare_decode_tensors / DecodeRuntimeStateLayout (standard_engine.cpp:128-150,
 * 1479-1572): binds the slot and sets the device state {kv_len, positions, step}.  kv_len =
 * tokens resident before the first decode step; mrope_pos = position of the first decoded
 * token on each axis (ignored for text models); step = response index the first decoded
 * token is written to (1 after a sampled prefill). */
EFM_API efm_status efm_b200_decode_begin(efm_b200_ctx* ctx, int32_t slot, int32_t kv_len,
                                         const int32_t mrope_pos[3], int32_t step);
/* Overwrites the device token slot (teacher forcing in tests). */
EFM_API efm_status efm_b200_set_token(efm_b200_ctx* ctx, int32_t token);
/* Replaces the decode loop body: Qwen2_5::decode_step + sampler + state advance, captured as
 * one CUDA graph when use_graph != 0 (standard_engine.cpp:772-859,975-1035).  Asynchronous. */
EFM_API efm_status efm_b200_decode_steps(efm_b200_ctx* ctx, int32_t n_steps, int32_t use_graph);
/* Captures the decode-step graph for a slot without running it (the reference captures during
 * warmup(): standard_engine.cpp:515-556).  Optional: decode_steps captures on first use. */
EFM_API efm_status efm_b200_capture_decode(efm_b200_ctx* ctx, int32_t slot);
/* One D2H copy of response tokens [first, first+n) + stream sync (standard_engine.cpp:1043-1057).
 * Also surfaces device-side status words (EFM_ERR_DEVICE_WAIT). */
EFM_API efm_status efm_b200_read_tokens(efm_b200_ctx* ctx, int32_t* host_out, int32_t first, int32_t n);
/* fp32 logits of the most recent forward ([vocab]); synchronises.  On a tensor-parallel context with imported peer
 * buffers and greedy sampling the ranks exchange only their maxima during a step, so this call gathers the ranks'
 * logits rows first: it is then a collective, to be made by every rank. */
EFM_API efm_status efm_b200_read_logits(efm_b200_ctx* ctx, float* host_out, int32_t n);
EFM_API efm_status efm_b200_synchronize(efm_b200_ctx* ctx);

/* ---- timing / accounting (CudaMetricRecorder, standard_engine.cpp:405-460) -------------- */
/* Records CUDA event `idx` (0..15) on the context stream. */
EFM_API efm_status efm_b200_event_record(efm_b200_ctx* ctx, int32_t idx);
EFM_API efm_status efm_b200_event_elapsed_ms(efm_b200_ctx* ctx, int32_t start_idx, int32_t stop_idx, float* ms);
/* Kernels launched by this context since creation (graph replays count their nodes). */
EFM_API efm_status efm_b200_launch_count(efm_b200_ctx* ctx, int64_t* count);
/* Runs n_steps decode steps as plain launches (no graph, no dependent-launch overlap) with an
 * event after every kernel and returns the summed device time per kernel kind in ms_out[7]:
 * qkv, attention, o_proj, gate_up, down_proj, lm_head, sampler.  Advances the decode state. */
EFM_API efm_status efm_b200_decode_breakdown(efm_b200_ctx* ctx, int32_t n_steps, float* ms_out);
/* Bytes of weights / KV one decode step must stream at the given kv_len (roofline numerator). */
EFM_API efm_status efm_b200_decode_step_bytes(efm_b200_ctx* ctx, int32_t kv_len, int64_t* bytes);

/* ---- single operators on caller-provided DEVICE buffers (parity tests per kernel; the
 * reference exposes the same granularity through its debug bindings, pybind_debug.cpp) ----- */
/* y[n] = W[n,:] . x.  x is bf16 [k]; with norm_w != NULL it is instead the fp32 residual stream and
 * x_used = bf16(rmsnorm(x) * norm_w).  With residual != NULL (fp32 [n]) the result is accumulated:
 * residual[n] += y[n]; else y_bf16[n] is written.
 * LinearLayer decode GEMV (src/operators/linear_impl.cu:457-469). */
EFM_API efm_status efm_b200_op_gemv(const void* w, const void* x, const void* norm_w, float eps,
                                    void* y_bf16, void* residual, int32_t n, int32_t k);
/* Consumer side of the tensor-parallel decode exchange on ONE GPU (no counterpart in the reference): the norm-prologue
 * GEMV whose input is resid + parts[0] + parts[1] + ... (rank order), parts being device [n_parts][k] 8-byte words
 * {fp32 value, count}.  Every word is re-read until it carries want_count, for at most wait_limit_us microseconds in
 * total; then y = W . bf16(rmsnorm(x) * norm_w) -> bf16 [n] and resid_out = x (fp32 [k], must differ from resid).
 * Returns EFM_ERR_DEVICE_WAIT when the wait ran out (outputs undefined; the device stays usable). */
EFM_API efm_status efm_b200_op_gemv_peer_consume(const void* w, const void* resid_f32, const void* norm_w, float eps,
                                                 const void* parts, int32_t n_parts, uint32_t want_count,
                                                 int64_t wait_limit_us, void* y_bf16, void* resid_out_f32, int32_t n,
                                                 int32_t k);
/* Y[m,n] = X[m,k] . W[n,k]^T (+bias[n]) -> bf16 (prefill linear; linear_impl.cu:457-469,482-706). */
EFM_API efm_status efm_b200_op_gemm(const void* x, const void* w, const void* bias, void* y_bf16,
                                    int32_t m, int32_t n, int32_t k);
/* Batch-1 GQA decode attention over a [max_tokens, kv, D] bf16 cache
 * (src/operators/attention_op.cu:1428-1466).  q: [q_heads, D] bf16 (already rotated). */
EFM_API efm_status efm_b200_op_decode_attention(const void* q, const void* k_cache, const void* v_cache,
                                                void* out_bf16, int32_t q_heads, int32_t kv_heads,
                                                int32_t head_dim, int32_t kv_len, int32_t max_tokens);
/* Same computation and arguments as efm_b200_op_decode_attention, for callers that must not
 * allocate device memory.  (No counterpart in the reference, whose attention call sizes a 32 MB
 * workspace itself.)  Some hosts of this library cannot call cudaMalloc at the point where they
 * need attention: a real-time control loop that promised its integrator a fixed memory footprint,
 * a plugin running inside another runtime's memory pool or inside a region where that runtime
 * forbids allocation, a process whose device memory was pre-partitioned at start-up.  This entry
 * point therefore keeps the split-KV scratch (partial outputs, softmax statistics, block tickets)
 * in a fixed array that is part of the library image: about 1 MB on every GPU that loads the
 * library, held until the process exits.  It calls no cudaMalloc / cudaFree and no allocating
 * library routine.
 * Limits: q_heads * head_dim <= 4096, q_heads <= 64, kv_heads <= 16 and q_heads / kv_heads <= 8;
 * larger shapes are refused with EFM_ERR_UNSUPPORTED (use efm_b200_op_decode_attention for those).
 * The first call on each device looks up the device address of that array (with that device
 * current) and caches it; the cache may be filled from several host threads at once.  The call
 * sets kernel attributes, runs on the default stream and synchronises it before returning, so it
 * must not be issued while a stream capture is active on the calling thread.
 * All calls share the one array and it keeps whatever the previous call left in it (the tickets
 * are re-zeroed at the start of every call): two calls whose kernels overlap on the GPU race on
 * it, so issue them one after the other (one host thread per device at a time). */
EFM_API efm_status efm_b200_op_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                                        void* out_bf16, int32_t q_heads, int32_t kv_heads,
                                                        int32_t head_dim, int32_t kv_len, int32_t max_tokens);
/* Causal GQA prefill attention, queries at cache rows [kv_offset, kv_offset+s)
 * (attention_op.cu:1221-1343).  q: [s, q_heads, D] bf16. */
EFM_API efm_status efm_b200_op_prefill_attention(const void* q, const void* k_cache, const void* v_cache,
                                                 void* out_bf16, int32_t s, int32_t kv_offset,
                                                 int32_t q_heads, int32_t kv_heads, int32_t head_dim);
/* INT8 ("SageAttention"-style) causal prefill attention, same arguments and layout as
 * efm_b200_op_prefill_attention; head_dim 64 or 128.  Keys are centred per kv head, Q and K quantised per
 * 128-token block and head (scale = max|x|/127), S from an exact int32 dot product, softmax in fp32, P and V in
 * fp16.  No source for it exists in the reference tree (README.md:23,456 mention it only). */
EFM_API efm_status efm_b200_op_sage_prefill_attention(const void* q, const void* k_cache, const void* v_cache,
                                                      void* out_bf16, int32_t s, int32_t kv_offset,
                                                      int32_t q_heads, int32_t kv_heads, int32_t head_dim);
/* Sampler on fp32 logits [vocab] -> one int32 (device).  SamplerLayer::forward
 * (src/layers/sampler.cu:146-299). */
EFM_API efm_status efm_b200_op_sample(const float* logits, int32_t vocab, const efm_sampling* s,
                                      uint32_t rng_step, int32_t* token_out);

/* Softmax attention where query row i sees the key rows [lo[i], hi[i]) (device int32 [s]); the
 * bidirectional windowed / full attention of the vision tower.  q, k, v are rows of `stride`
 * elements with head h at column h*D (q, k, v may be three column ranges of one fused qkv
 * buffer); out: [s, heads*D] bf16.  head_dim 64, 80 or 128.  No counterpart in the reference. */
EFM_API efm_status efm_b200_op_segment_attention(const void* q, const void* k, const void* v, void* out_bf16,
                                                 const int32_t* lo, const int32_t* hi, int32_t s,
                                                 int32_t heads, int32_t head_dim, int32_t stride);

/* ---- Qwen2.5-VL vision encoder ------------------------------------------------------------
 * The reference has no vision tower: callers run one elsewhere and pass its output through
 * Request.embedding (examples/qwen2.5-vl-3b-instruct/generate.py:3, embed_head.cu:63-132).
 * These entry points produce exactly that tensor on the device, on the stream of the text
 * context they were created from, so that encode -> efm_b200_prefill(embeds, EFM_MEM_DEVICE)
 * needs no copy and no host synchronisation.  Algorithm: the published Qwen2.5-VL encoder
 * (patch embedding, window-major token order, 2-D rotary, windowed / full bidirectional
 * attention, SiLU-gated MLP, 2x2 merger). */
typedef struct efm_vit_desc {
    int32_t struct_size;          /* = sizeof(efm_vit_desc) */
    int32_t depth;
    int32_t hidden;               /* heads * head_dim */
    int32_t heads;                /* head_dim 64, 80 or 128 */
    int32_t intermediate;         /* any multiple of 4 (zero-padded to 64 inside) */
    int32_t out_hidden;           /* width of the produced embeddings = LLM hidden */
    int32_t patch;                /* 14 */
    int32_t temporal_patch;       /* 2 */
    int32_t in_channels;          /* 3 */
    int32_t merge;                /* 2: merge x merge patches per produced token */
    int32_t window;               /* 112 (pixels) */
    int32_t n_fullatt;            /* number of layers with full attention, <= 8 */
    int32_t fullatt[8];           /* their indices */
    float rms_eps;
    float rope_theta;
    int32_t max_patches;          /* capacity of one encode call */
} efm_vit_desc;

typedef struct efm_b200_vit efm_b200_vit;

/* The encoder lives on ctx's device and stream and reports errors through
 * efm_b200_last_error(ctx); destroy it before ctx. */
EFM_API efm_status efm_b200_vit_create(efm_b200_ctx* ctx, const efm_vit_desc* desc, efm_b200_vit** out);
EFM_API efm_status efm_b200_vit_destroy(efm_b200_vit* vit);
/* HF tensor names "visual.*" (patch_embed.proj, blocks.N.{norm1,norm2,attn.qkv,attn.proj,
 * mlp.gate_proj,mlp.up_proj,mlp.down_proj}, merger.{ln_q,mlp.0,mlp.2}); bf16, whole tensors. */
EFM_API efm_status efm_b200_vit_set_weight(efm_b200_vit* vit, const char* hf_name, const void* data,
                                           const int64_t* shape, int32_t ndim, int32_t dtype,
                                           int32_t mem_kind);
EFM_API efm_status efm_b200_vit_finalize_weights(efm_b200_vit* vit);
/* pixels: bf16 [n_patches, in_channels*temporal_patch*patch*patch] in the image processor's row
 * order (every merge*merge consecutive rows are one block), host or device per pixels_mem.
 * grid_thw: host int32 [n_grids, 3] patch grids (frames, rows, columns); n_patches = sum t*h*w.
 * out: bf16 [n_patches / merge^2, out_hidden], host or device per out_mem, in the original
 * (row-major merged-grid) order.  Asynchronous on the context's stream when out is on the device. */
/* Host-only (no GPU needed): the plan efm_b200_vit_encode derives from the patch grids.  For n_patches =
 * sum t*h*w and n_merged = n_patches / merge^2 it fills (any pointer may be NULL):
 *   order[n_merged]   window-major order: position i holds merged token order[i] of the row-major input;
 *   pos_h/pos_w[n_patches]  patch row / column (inside its frame) of the patch at each permuted position;
 *   win_lo/win_hi[n_patches]  attention range of each permuted position in the windowed layers;
 *   full_lo/full_hi[n_patches] the same for the full-attention layers (the patch's frame).
 * Returns EFM_ERR_INVALID_ARGUMENT for grids that are not positive multiples of the merge size. */
EFM_API efm_status efm_b200_vit_plan(const efm_vit_desc* desc, const int32_t* grid_thw, int32_t n_grids,
                                     int32_t* order, int32_t* pos_h, int32_t* pos_w, int32_t* win_lo,
                                     int32_t* win_hi, int32_t* full_lo, int32_t* full_hi);
EFM_API efm_status efm_b200_vit_encode(efm_b200_vit* vit, const void* pixels, int32_t pixels_mem,
                                       const int32_t* grid_thw, int32_t n_grids, void* out,
                                       int32_t out_mem);

/* ---- SmolVLA-shaped action chunk ----------------------------------------------------------
 * The reference describes this model (doc/smolvla_architecture.md) but ships no code for it; its
 * closest entry point is the trajectory planner's Euler loop
 * (src/engine/tasks/trajectory_planning/trajectory_planner_engine.cpp:298-318, edge-fm.h:49-75 plan()).
 * One call = one action chunk: SigLIP-style vision tower + pixel-shuffle connector on n_images square
 * images, Llama-style backbone over [image tokens | prompt | state], action expert with alternating
 * self / cross attention over the backbone's KV rows, `steps` flow-matching Euler steps from `noise`.
 * The object owns its device buffers and stream; it needs no text context. */
typedef struct efm_vla_desc {
    int32_t struct_size;          /* = sizeof(efm_vla_desc) */
    int32_t image_size, patch, vit_layers, vit_hidden, vit_heads, vit_mlp;   /* vit_hidden = vit_heads * 64 */
    int32_t shuffle, n_images;    /* pixel-shuffle factor; (image_size / patch) % shuffle == 0 */
    int32_t hidden, layers, q_heads, kv_heads, head_dim, mlp;  /* backbone; head_dim 64; layers even; the expert has the same heads and depth */
    int32_t vocab, lang_tokens;
    int32_t expert_hidden, expert_mlp;
    int32_t state_dim, action_dim, chunk, steps;
    float rope_theta, rms_eps, ln_eps;
} efm_vla_desc;

typedef struct efm_b200_vla efm_b200_vla;

EFM_API efm_status efm_b200_vla_create(const efm_vla_desc* desc, int32_t device, efm_b200_vla** out);
EFM_API efm_status efm_b200_vla_destroy(efm_b200_vla* vla);
EFM_API const char* efm_b200_vla_last_error(const efm_b200_vla* vla);
/* bf16 tensors by name: vit.patch.{weight,bias}, vit.pos, vit.N.{ln1,ln2,q,k,v,o,fc1,fc2}.{weight,bias},
 * vit.post_ln.{weight,bias}, connector.weight, embed, state_proj.{weight,bias},
 * vlm.N.{norm1,norm2} and vlm.N.{q,k,v,o,gate,up,down}.weight, the same under expert.N. (k / v of the odd,
 * cross-attention layers are [kv_dim, kv_dim]), expert.norm, action_in / time_in / time_out /
 * action_out .{weight,bias}.  Linear weights are [out, in] row-major as in the checkpoint. */
EFM_API efm_status efm_b200_vla_set_weight(efm_b200_vla* vla, const char* name, const void* data,
                                           const int64_t* shape, int32_t ndim, int32_t dtype, int32_t mem_kind);
EFM_API efm_status efm_b200_vla_finalize_weights(efm_b200_vla* vla);
/* images fp32 [n_images, 3, image_size, image_size] (already normalised), lang_ids int32 [lang_tokens],
 * state fp32 [state_dim], noise fp32 [chunk, action_dim]; actions_out fp32 [chunk, action_dim].  All five
 * on the host or all on the device per mem_kind; a NULL input keeps what the previous call uploaded.
 * Synchronous: returns when actions_out is written.  The first call launches kernel by kernel, later
 * calls replay one captured graph. */
EFM_API efm_status efm_b200_vla_chunk(efm_b200_vla* vla, const float* images, const int32_t* lang_ids,
                                      const float* state, const float* noise, int32_t mem_kind,
                                      float* actions_out);
/* One chunk on the inputs already resident from an earlier efm_b200_vla_chunk call, enqueued on the
 * object's stream without synchronising (for device-side timing); the stream for events. */
EFM_API efm_status efm_b200_vla_enqueue(efm_b200_vla* vla);
EFM_API efm_status efm_b200_vla_stream(efm_b200_vla* vla, void** stream_out);
/* Device time of the four phases of one chunk (vision, prefix, bridge, denoise), launched kernel by kernel on
 * the resident inputs with events in between: ms4[4].  A profiling aid; the graph replay is faster. */
EFM_API efm_status efm_b200_vla_phase_ms(efm_b200_vla* vla, float* ms4);
/* kernels launched so far / per chunk (graph replays count their kernel nodes) */
EFM_API efm_status efm_b200_vla_launch_count(const efm_b200_vla* vla, int64_t* total, int64_t* per_chunk);

#ifdef __cplusplus
}
#endif
#endif /* EFM_B200_H_ */
