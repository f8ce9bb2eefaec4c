/*
 * vuib200.h - C ABI of libvuib200: Vui Nano's per-codec-frame decode step as
 * hand-written CUDA for sm_100a.
 *
 * The reference (fluxions-ai/vui) is pure Python over PyTorch: it has no FFI for
 * this path, so each entry point cites the Python function whose device work it
 * replaces (paths relative to that project).  The Python shim in
 * vui_b200/engine.py keeps the reference's Engine / Row / GenConfig surface and
 * calls these through ctypes.
 *
 * Conventions
 *  - every function returns a VuibStatus (0 = OK, negative = error); nothing
 *    throws, aborts or exits; vuib_last_error() gives the text of the last error.
 *  - all "dev" pointers are DEVICE pointers borrowed from the caller (torch
 *    tensors); the library never allocates or frees device memory, and never
 *    synchronises the device unless a function says so.
 *  - every kernel is launched on the cudaStream_t the caller passes (as void*),
 *    so the calls can be captured into a CUDA graph and replayed once per frame.
 *  - a handle is not thread-safe; use one host thread per engine.
 *  - matrices are bf16, row-major (out_features, in_features), as torch stores
 *    nn.Linear.weight.  Codes are int64.  KV layout is the reference's
 *    FlashKVCache: (slots, max_seq, n_kv_heads, head_dim) bf16 per layer plus one
 *    shared int32 seq_lens[slots]  (src/vui/model.py:71-99, 473-495).
 */
#ifndef VUIB200_H
#define VUIB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VUIB_ABI_VERSION 1
#define VUIB_MAX_LAYERS 64

typedef enum VuibStatus {
    VUIB_OK = 0,
    VUIB_ERR_NULL = -1,        /* a required pointer is NULL */
    VUIB_ERR_SHAPE = -2,       /* unsupported model shape */
    VUIB_ERR_RANGE = -3,       /* batch / row count / slot / length out of range */
    VUIB_ERR_UNBOUND = -4,     /* weights, KV, rope table or workspace not bound yet */
    VUIB_ERR_CUDA = -5,        /* a CUDA runtime call failed (text in last_error) */
    VUIB_ERR_WORKSPACE = -6,   /* workspace too small or misaligned */
    VUIB_ERR_DEVICE_FLAG = -7  /* a kernel recorded a bad slot / position / code, or a barrier timeout */
} VuibStatus;

/* Model + engine shape.  Mirrors vui.config.VuiConfig (src/vui/config.py:16-54)
 * plus the sizes Engine.__init__ fixes (src/vui/engine.py:294-346). */
typedef struct VuibConfig {
    int32_t d_model, n_layers, n_heads, n_kv_heads, head_dim, ffn;
    int32_t n_quantizers, codebook_size;
    int32_t rq_d_model, rq_n_layers, rq_n_heads, rq_ffn;
    float norm_eps;     /* backbone RMSNorm eps (1e-5) */
    float rq_norm_eps;  /* depth-transformer RMSNorm eps (1e-6) */
    int32_t n_slots;    /* KV slots = max_rows + 1 (spare slot = padding target) */
    int32_t max_seq;    /* positions per slot */
    int32_t max_rows;   /* most rows (streams) in one decode step */
    int32_t max_prefill_rows; /* most rows (positions) in one prefill call */
} VuibConfig;

/* Borrowed device pointers to the weights; names follow the reference state dict
 * (src/vui/mlx/tts/weights.py:121-192 lists the keys). */
typedef struct VuibWeights {
    const void* audio_emb;   /* audio_emb.embedding.weight (Q*CS, d) */
    const void* codec_head;  /* codec_head.weight (CS, d) */
    const void* eos_w;       /* eos_head.weight (1, d) */
    const void* eos_b;       /* eos_head.bias (1) */
    const void* final_norm;  /* decoder.norm.weight (d) */
    const void* attn_norm[VUIB_MAX_LAYERS];
    const void* wqkv[VUIB_MAX_LAYERS];      /* ((H+2Hkv)*hd, d), rows q|k|v */
    const void* out_proj[VUIB_MAX_LAYERS];  /* (d, d) */
    const void* mlp_norm[VUIB_MAX_LAYERS];
    const void* w1[VUIB_MAX_LAYERS];        /* (ffn, d) */
    const void* w3[VUIB_MAX_LAYERS];        /* (ffn, d) */
    const void* w2[VUIB_MAX_LAYERS];        /* (d, ffn) */
    const void* rq_backbone_proj;  /* (rd, d) */
    const void* rq_code_emb;       /* ((Q-1)*CS, rd) */
    const void* rq_pos_emb;        /* (Q, rd) */
    const void* rq_head;           /* head_W (Q-1, CS, rd) */
    const void* rq_norm;           /* (rd) */
    const void* rq_attn_norm[VUIB_MAX_LAYERS];
    const void* rq_wqkv[VUIB_MAX_LAYERS];   /* (3*rd, rd) */
    const void* rq_out_proj[VUIB_MAX_LAYERS];
    const void* rq_mlp_norm[VUIB_MAX_LAYERS];
    const void* rq_w1[VUIB_MAX_LAYERS];
    const void* rq_w3[VUIB_MAX_LAYERS];
    const void* rq_w2[VUIB_MAX_LAYERS];
} VuibWeights;

/* Sampling controls for one depth step.  Copied to the device by
 * vuib_set_sampling(), so a captured graph picks up new values on replay. */
typedef struct VuibSampling {
    float temperature;     /* cb0 and depth codebooks (engine.py:857, model.py:957) */
    int32_t top_k_cb0;     /* 1 = greedy (first index on ties), 0 = whole distribution */
    int32_t top_k_rq;      /* 1 = greedy; the reference captures 100 (engine.py:395-397) */
    float rep_penalty;     /* <= 1 disables (engine.py:571-590) */
    int32_t rep_window;    /* 0 = counts never expire (engine.py:606-616) */
    int32_t n_codebooks;   /* 0 = all Q; else emit Q' codes, rest zero (engine.py:473-479) */
    uint64_t seed;         /* Philox key; draws are keyed (seed, slot, frame, codebook) */
} VuibSampling;

typedef struct VuibEngine VuibEngine;

int32_t vuib_abi_version(void);

/* Validates the shape and creates a handle (host memory only).
 * Replaces the bookkeeping half of Engine._setup_graphs (engine.py:375-432). */
int32_t vuib_create(const VuibConfig* cfg, VuibEngine** out);
int32_t vuib_destroy(VuibEngine* e);
int32_t vuib_last_error(VuibEngine* e, char* buf, size_t n);

/* Scratch for activations, attention partials, depth-transformer KV, sampling
 * state.  The caller allocates `bytes` (256-byte aligned), ZEROES it once, and
 * binds it; it must outlive the handle's use. */
int32_t vuib_workspace_bytes(VuibEngine* e, size_t* bytes);
int32_t vuib_bind_workspace(VuibEngine* e, void* dev, size_t bytes);

int32_t vuib_bind_weights(VuibEngine* e, const VuibWeights* w);
/* k[l], v[l]: (n_slots, max_seq, n_kv_heads, head_dim) bf16; seq_lens: int32[n_slots].
 * Same tensors the reference keeps in model.decoder.flash_kv_caches (model.py:473-495),
 * so its KV save/load code (serving/stream/tts_worker.py:885-1028) keeps working. */
int32_t vuib_bind_kv(VuibEngine* e, void* const* k_dev, void* const* v_dev, int32_t* seq_lens_dev);
/* (max_seq, head_dim, 2) bf16 [cos, sin] table as precompute_freqs_cis builds it
 * (src/vui/rope.py:60-77) and Vui.bfloat16() casts it. */
int32_t vuib_bind_rope(VuibEngine* e, const void* freqs_cis_dev);

/* Copies *s to the device-side control block (async on `stream`). */
int32_t vuib_set_sampling(VuibEngine* e, const VuibSampling* s, void* stream);

/* Optional per-row statistics of the cb0 draw (NULL disables): cb0_stats_dev is (max_rows, 2) fp32 on
 * the device; every frame row r gets [2r] = entropy in nats and [2r+1] = largest probability of
 * softmax(repetition-penalised cb0 logits / temperature) over the whole codebook.  Replaces
 * _entropy_top1 of Engine._stream_row (engine.py:1369-1372), which the streaming gate averages over
 * the first frames of a chunk (engine.py:1418-1424, 1455-1460, 1488-1516).  Set it before frames are
 * captured in a graph. */
int32_t vuib_set_stats(VuibEngine* e, float* cb0_stats_dev);

/* Optional debug taps for the parity tests (NULL disables each):
 *  layer_hidden: (n_layers, max_rows, d) bf16 - residual stream after each block
 *  rq_logits:    (max_rows, Q-1, CS) bf16     - depth-head logits per codebook   */
int32_t vuib_set_taps(VuibEngine* e, void* layer_hidden_dev, void* rq_logits_dev);

/* Prefill: run n_rows embeddings through the backbone, appending K/V.
 * Replaces Engine._prefill_emb (engine.py:674-694) for any number of slots at once.
 *  row_slot/row_pos: int32[n_rows] - slot and position of each row; rows of one
 *      slot must carry consecutive positions starting at that slot's length.
 *  emb: (n_rows, d) bf16;  hidden_out: (n_rows, d) bf16 final-norm output.
 * Does not touch seq_lens (the caller adds the segment lengths, as the reference
 * does on the host).  Slots and positions outside the cache are clamped and recorded in the
 * device flag, so K/V are never written out of bounds. */
int32_t vuib_prefill(VuibEngine* e, int32_t n_rows, const int32_t* row_slot_dev,
                     const int32_t* row_pos_dev, const void* emb_dev, void* hidden_out_dev,
                     void* stream);

/* One backbone decode step for B rows.  Replaces Engine._backbone_decode_body(_b)
 * (engine.py:434-449, 485-502): embeds codes_in (gather-sum, model.py:559-563),
 * 24 blocks at position seq_lens[slot], final norm, codec_head, eos_head, then
 * seq_lens[slot[r]] += seq_inc[r] (1 when seq_inc is NULL).
 *  slots: int32[B]; codes_in: int64 (B, Q); hidden_out (B, d), cb0_out (B, CS),
 *  eos_out (B, 1): bf16. */
int32_t vuib_backbone_step(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                           const int32_t* seq_inc_dev, const int64_t* codes_in_dev,
                           void* hidden_out_dev, void* cb0_out_dev, void* eos_out_dev,
                           void* stream);

/* codec_head + eos_head on an already final-normed hidden (B, d): the frame-0
 * path, model.codec_head(hidden) at engine.py:929, 1152, 1414. */
int32_t vuib_heads(VuibEngine* e, int32_t B, const void* hidden_dev, void* cb0_out_dev,
                   void* eos_out_dev, void* stream);

/* Depth step: sample cb0 from cb0_logits (Engine._sample_cb0 + _rep_apply/_rep_push,
 * engine.py:571-590, 855-863) then the RQ depth transformer over codebooks 1..Q-1
 * (RQTransformer._generate_graph_body_kv, model.py:908-986) with no host round
 * trip between codebooks.  Writes codes_out (B, Q) int64 and eos_prob_out (B) f32
 * = sigmoid(eos logit) when both eos pointers are given.
 *  first_frame != 0 samples cb0 from the whole distribution (engine.py:936-937). */
int32_t vuib_depth_step(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                        const void* hidden_dev, const void* cb0_logits_dev,
                        const void* eos_logit_dev, int32_t first_frame,
                        int64_t* codes_out_dev, float* eos_prob_out_dev, void* stream);

/* backbone step + depth step: one whole frame; codes_io holds frame k-1 on entry
 * and frame k on return, so replaying the captured call generates a stream. */
int32_t vuib_decode_frame(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                          const int32_t* seq_inc_dev, int64_t* codes_io_dev,
                          void* hidden_out_dev, void* cb0_out_dev, void* eos_out_dev,
                          float* eos_prob_out_dev, void* stream);

/* One whole frame from and to HOST memory, as one CUDA-graph launch: what the per-frame body of `_stream_row`
 * (engine.py:1450-1546: replay the frame, read the codes and the EOS probability back) costs a serving loop.
 *
 * vuib_frame_host_capture records, for this B and these device buffers, the graph
 *   [pinned staging -> codes_io (only when with_h2d != 0)] -> vuib_decode_frame -> [codes_io, eos_prob -> pinned staging]
 * on `stream` (a stream of the caller's, not the default stream).  The kernels must have run once before (module
 * loading cannot happen inside a capture): call vuib_decode_frame, or replay a captured one, first.  Capturing again
 * for the same (B, with_h2d) replaces the earlier graph.  The staging buffers and graphs are freed by vuib_destroy.
 *
 * vuib_frame_host copies codes_in_host (B, Q) int64 into the staging buffer (with_h2d != 0), launches the graph,
 * waits for it on `stream` and copies the frame's codes (B, Q) and EOS probabilities (B, may be NULL) out.  The
 * device buffers named at capture must still be alive.  Returns VUIB_ERR_UNBOUND without a captured graph. */
int32_t vuib_frame_host_capture(VuibEngine* e, int32_t B, int32_t with_h2d, const int32_t* slots_dev,
                                const int32_t* seq_inc_dev, int64_t* codes_io_dev, void* hidden_out_dev,
                                void* cb0_out_dev, void* eos_out_dev, float* eos_prob_out_dev, void* stream);
int32_t vuib_frame_host(VuibEngine* e, int32_t B, int32_t with_h2d, const int64_t* codes_in_host,
                        int64_t* codes_out_host, float* eos_prob_out_host, void* stream);

/* Decode attention alone over layer `layer` of the bound KV cache: the device work of the
 * flash_attn_with_kvcache call (MHA.forward_flash, model.py:247-257) minus the append, which
 * the QKV kernel has already done.  Row r attends keys [0, row_pos[r]] of slot row_slot[r];
 * GQA (n_heads / n_kv_heads query heads per KV head), scale 1/sqrt(head_dim), fp32 softmax.
 *  q, out: (n_rows, n_heads*head_dim) bf16, q with RoPE applied; n_rows <= max(max_rows,
 *  max_prefill_rows).  Uses the bound workspace for its split-KV partial results.
 *  A slot outside [0, n_slots) or a position outside [0, max_seq) is clamped into the cache and
 *  recorded in the device flag (vuib_check_device_flag); nothing is read out of bounds. */
int32_t vuib_attention(VuibEngine* e, int32_t layer, int32_t n_rows, const void* q_dev,
                       const int32_t* row_slot_dev, const int32_t* row_pos_dev, void* out_dev,
                       void* stream);

/* vuib_attention for callers that cannot allocate device memory.  It has no counterpart in
 * the reference; it exists for hosts of this library that may not call cudaMalloc: a real-time
 * audio thread that must never wait on the driver's allocator, or a plug-in inside a server
 * that owns all device memory through its own pool.  It needs no handle and no workspace: the
 * split-KV partial results live in a fixed array inside the library (about 529 KB, held by every
 * GPU that loads the library until the process exits), and it calls neither cudaMalloc nor
 * cudaFree nor any allocating routine.
 *  Limits: n_rows <= 8, max_seq <= 2048, n_heads <= 16 with 1 or 2 query heads per kv head,
 *  head_dim 64.  Larger sizes return VUIB_ERR_RANGE with the reason in `err`.
 *  k_cache / v_cache: (slots, max_seq, n_kv_heads, 64) bf16 of ONE layer; q, out: (n_rows,
 *  n_heads*64) bf16; row r attends keys [0, row_pos[r]] of slot row_slot[r].
 *  Positions outside [0, max_seq) are clamped on the device and negative slots read slot 0; the
 *  number of slots is not known here, so a slot past the end of the caller's cache cannot be caught.
 *  The first call on a device looks up the array's device address (cudaGetSymbolAddress), so
 *  make that call before starting any stream capture.  All calls share the one array: it keeps
 *  the last call's contents (the call clears what it needs zeroed), and two calls that overlap
 *  on the GPU (different streams) race; keep them on one stream or order them.
 *  err / err_len: optional buffer for the error text. */
int32_t vuib_attention_noalloc(int32_t n_heads, int32_t n_kv_heads, int32_t max_seq, int32_t n_rows,
                               const void* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                               const int32_t* row_slot_dev, const int32_t* row_pos_dev, void* out_dev,
                               void* stream, char* err, size_t err_len);

/* Gather-sum of codec codes alone: out[r] = sum_q audio_emb[q*CS + codes[r,q]]
 * (AudioEmbedding.forward, model.py:559-563; Engine._audio_emb, engine.py:705-709).
 * codes: int64 (n_rows, Q); out: bf16 (n_rows, d).  Feeds a prefill of audio frames. */
int32_t vuib_embed_codes(VuibEngine* e, int32_t n_rows, const int64_t* codes_dev, void* out_dev,
                         void* stream);

/* The sampler alone on caller-supplied logits (B, CS) bf16: codebook 0 follows
 * Engine._sample_cb0 (+ repetition penalty), codebooks >= 1 the depth-transformer
 * rule (model.py:955-962).  Writes one int64 per row and advances the slot's
 * draw counter.  Used by the distribution tests. */
int32_t vuib_sample_rows(VuibEngine* e, int32_t B, const int32_t* slots_dev, const void* logits_dev,
                         int32_t codebook, int64_t* codes_out_dev, void* stream);

/* Single fused ops for parity tests.  With an identity matrix as w the product passes its staged
 * input through exactly, so the outputs can be held bit for bit against the reference's modules:
 *  vuib_debug_norm_linear: out (n_rows, n_out) = bf16(W . RMSNorm(x) * norm_w)   (RMSNorm.forward,
 *      src/vui/model.py:292-297, as staged in front of Wqkv / w1 / w3); x (n_rows, d_model).
 *  vuib_debug_linear_rope: out (n_rows, d_model) = RoPE(bf16(W . x)) at position row_pos[r], every
 *      64 columns one head (apply_rotary_emb, src/vui/rope.py:23-57); W (d_model, d_model).
 * tensor_cores = 0 runs the weight-streaming GEMV kernels, 1 the tcgen05 GEMM kernels
 * (n_out a multiple of 128).  n_rows <= max(max_rows, max_prefill_rows). */
int32_t vuib_debug_norm_linear(VuibEngine* e, int32_t n_rows, const void* x_dev, const void* norm_w_dev,
                               const void* w_dev, int32_t n_out, void* out_dev, int32_t tensor_cores,
                               void* stream);
int32_t vuib_debug_linear_rope(VuibEngine* e, int32_t n_rows, const void* x_dev, const void* w_dev,
                               const int32_t* row_pos_dev, void* out_dev, int32_t tensor_cores, void* stream);

/* Clears the repetition-penalty state (counts + rolling history) of one slot, or
 * of every slot when slot == -1: Engine._rep_reset / _rep_reset_slot
 * (engine.py:555-569, 594-595).  Async on `stream`. */
int32_t vuib_rep_reset(VuibEngine* e, int32_t slot, void* stream);

/* Copies a slot's repetition-penalty state out of the workspace: counts_out_dev gets codebook_size
 * fp32 counts (how often each cb0 code sits in the window), filled_out_dev (optional) the number of
 * codes the rolling window holds.  The reference keeps these as Engine._rep_counts / _rep_filled
 * (engine.py:555-569), which its serving layer logs (serving/stream/tts_worker.py:646-653).  Async on
 * `stream`; both outputs are device pointers. */
int32_t vuib_rep_state(VuibEngine* e, int32_t slot, float* counts_out_dev, int32_t* filled_out_dev, void* stream);

/* Zeroes the mutable sampler / bookkeeping state in the workspace: per-slot draw counters,
 * repetition-penalty state, the device error flag.  Weights, KV and lengths are untouched.
 * (The reference has no equivalent: its draws come from torch's global generator.) */
int32_t vuib_reset_state(VuibEngine* e, void* stream);

/* Profiling aid: when the environment variable VUIB_TRACE is set, CTA (0,0) of a tensor-core GEMM
 * launch records device-clock stamps (ns) at its pipeline stages.  Copies the first n_stamps (<= 64)
 * stamps of the last such launch to out_host.  Synchronous. */
int32_t vuib_read_trace(VuibEngine* e, uint64_t* out_host, int32_t n_stamps);

/* Every wait inside a kernel (the tile counter on which the K-splits of a tensor-core GEMM meet, its
 * mbarrier pipeline) gives up after a bounded number of polls, records the device flag and lets the
 * kernel finish; this sets that bound (default 2^22 polls, at least 16).  A frame that reported the
 * flag is followed by vuib_reset_state before the handle is used again. */
int32_t vuib_set_wait_limit(VuibEngine* e, uint32_t polls);

/* Test hook for the bound above: presets the arrival counters so that the next tensor-core GEMM
 * launch sees one arrival fewer than it waits for.  Its wait runs out, the flag is recorded, the
 * kernel returns.  Nothing faults or hangs.  Synchronises `stream`. */
int32_t vuib_debug_withhold_arrival(VuibEngine* e, void* stream);

/* Position-only rewind / reset (engine.py:651-654).  Synchronous small copies. */
int32_t vuib_set_seq_len(VuibEngine* e, int32_t slot, int32_t len);
int32_t vuib_get_seq_len(VuibEngine* e, int32_t slot, int32_t* len);

/* Reads and clears the device error flag (bad slot / position / code seen by a
 * kernel).  Synchronises `stream`. */
int32_t vuib_check_device_flag(VuibEngine* e, void* stream);

/* Kernel launches issued by this handle since creation (for benchmarks). */
int64_t vuib_launch_count(VuibEngine* e);

/* ---------------------------------------------------------------------------
 * Streaming codec decode: one frame of 16 codes -> 1920 samples at 24 kHz, fp32.
 * Replaces the device work of QwenCodecDecoder's single-frame streaming forward
 * (src/vui/qwen_codec.py:1191-1224, captured as a CUDA graph by setup_streaming_graph,
 * 1138-1189) as CodecCtx.decode_frame drives it (625-657); call site
 * Engine._stream_decode_frame (src/vui/engine.py:1537-1546).
 * All tensors fp32.  Weight pointers are borrowed; layouts are torch's unless noted.
 * ------------------------------------------------------------------------- */
#define VUIB_CODEC_LAYERS 8
#define VUIB_CODEC_STAGES 2
#define VUIB_CODEC_BLOCKS 4

/* Fixed architecture of the 12.5 Hz decoder (qwen_codec.py:1080-1125); the fields exist so that a
 * mismatching checkpoint is refused instead of misread. */
typedef struct VuibCodecConfig {
    int32_t n_q;            /* 16 codebooks: 1 semantic + 15 acoustic */
    int32_t codebook_size;  /* 2048 */
    int32_t codebook_dim;   /* 256 */
    int32_t vq_dim;         /* 512 */
    int32_t latent_dim;     /* 1024 */
    int32_t d_model;        /* 512 */
    int32_t n_layers;       /* 8 */
    int32_t n_heads;        /* 16 (x head_dim 64 = 1024) */
    int32_t mlp_dim;        /* 1024 */
    int32_t max_seq;        /* 250 transformer positions */
    int32_t decoder_dim;    /* 1536 */
    int32_t rates[VUIB_CODEC_BLOCKS];  /* 8, 5, 4, 3 */
    float norm_eps;         /* RMSNorm eps 1e-6 */
} VuibCodecConfig;

typedef struct VuibSnakeW {   /* SnakeBeta (qwen_codec.py:820-829), per channel, precomputed: */
    const float* ea;          /*   exp(alpha) */
    const float* ib;          /*   1 / (exp(beta) + 1e-9) */
} VuibSnakeW;
typedef struct VuibConvW { const float* w; const float* b; } VuibConvW;
typedef struct VuibCodecLayerW {   /* DecTransformerBlock (qwen_codec.py:882-974) */
    const float* ln1;         /* input_layernorm.weight (512) */
    const float* wqkv;        /* q_proj | k_proj | v_proj weights stacked by rows: (3072, 512) */
    const float* wo;          /* o_proj.weight (512, 1024) */
    const float* attn_scale;  /* (512) */
    const float* ln2;         /* post_attention_layernorm.weight */
    const float* gate;        /* gate_proj.weight (1024, 512) */
    const float* up;          /* up_proj.weight (1024, 512) */
    const float* down;        /* down_proj.weight (512, 1024) */
    const float* mlp_scale;   /* (512) */
} VuibCodecLayerW;
typedef struct VuibUpStageW {      /* upsample[i] = [CausalTransConv1d k=2 s=2, ConvNeXtBlock] (1103-1113) */
    VuibConvW up;             /* w re-laid as rows (co, j): (1024 * 2, 1024) = weight.permute(1, 2, 0); b (1024) */
    VuibConvW dw;             /* dwconv.conv.weight (1024, 7), bias (1024) */
    const float* ln_w; const float* ln_b;
    VuibConvW pw1;            /* (4096, 1024), (4096) */
    VuibConvW pw2;            /* (1024, 4096), (1024) */
    const float* gamma;       /* (1024) */
} VuibUpStageW;
/* The tiled kernel wants a weight per tile of 96 output rows, K-major inside the tile:
 * [rows / 96][C_in][taps][96], i.e. weight.view(rows / 96, 96, C_in, taps).permute(0, 2, 3, 1). */
typedef struct VuibResUnitW {      /* DecoderResUnit (851-860) */
    VuibSnakeW act1; VuibConvW conv1;   /* (C, C, 7) re-laid as above, dilation 1 / 3 / 9 */
    VuibSnakeW act2; VuibConvW conv2;   /* (C, C, 1) re-laid as above */
} VuibResUnitW;
typedef struct VuibDecBlockW {     /* DecoderBlock (863-879) */
    VuibSnakeW act;
    VuibConvW up;             /* rows (co, k) = (Cout * 2 * rate) over Cin.  Block 0 (4 columns per frame, row kernel):
                                 (rows, Cin) = weight.permute(1, 2, 0); blocks 1..3 (tiled kernel): re-laid as above with
                                 one tap; b (Cout) */
    VuibResUnitW res[3];
} VuibDecBlockW;
typedef struct VuibCodecWeights {
    const float* codebook[16];     /* quantizer.semantic.codebooks.0.embed, then acoustic 0..14: (2048, 256) */
    const float* sem_proj;         /* quantizer.semantic.output_proj.weight (512, 256) */
    const float* acq_proj;         /* quantizer.acoustic.output_proj.weight (512, 256) */
    VuibConvW pre_conv;            /* (1024, 512, 3), (1024) */
    VuibConvW in_proj;             /* pre_transformer.input_proj (512, 1024), (512) */
    VuibCodecLayerW layer[VUIB_CODEC_LAYERS];
    const float* norm;             /* pre_transformer.norm.weight (512) */
    VuibConvW out_proj;            /* (1024, 512), (1024) */
    const float* rope_cos;         /* (max_seq, 64) as RoPE.forward builds them (qwen_codec.py:161-171) */
    const float* rope_sin;
    VuibUpStageW stage[VUIB_CODEC_STAGES];
    VuibConvW dec_in;              /* decoder.0 (1536, 1024, 7), (1536) */
    VuibDecBlockW block[VUIB_CODEC_BLOCKS];
    VuibSnakeW final_act;          /* decoder.5 (96) */
    VuibConvW final_conv;          /* decoder.6 (1, 96, 7), (1) */
} VuibCodecWeights;

typedef struct VuibCodec VuibCodec;

int32_t vuib_codec_create(const VuibCodecConfig* cfg, VuibCodec** out);
int32_t vuib_codec_destroy(VuibCodec* c);
int32_t vuib_codec_last_error(VuibCodec* c, char* buf, size_t n);
/* Streaming state (convolution histories, transposed-convolution partials, transformer KV and position)
 * and activations live in one caller-allocated block, 256-byte aligned, zeroed once. */
int32_t vuib_codec_workspace_bytes(VuibCodec* c, size_t* bytes);
int32_t vuib_codec_bind_workspace(VuibCodec* c, void* dev, size_t bytes);
int32_t vuib_codec_bind_weights(VuibCodec* c, const VuibCodecWeights* w);
/* Fresh streaming state: what entering decoder.streaming(1) / reset_streaming() does to every
 * StreamingModule (qwen_codec.py:74-90, 122-138, 1011-1032).  Async on `stream`. */
int32_t vuib_codec_reset(VuibCodec* c, void* stream);
/* One frame: codes_dev int64[n_q] (n_q <= 16: fewer codebooks decode coarser audio, engine.py:1544-1545),
 * audio_out_dev float[1920], clamped to [-1, 1].  Advances the streaming state.  Capturable in a graph. */
int32_t vuib_codec_decode_frame(VuibCodec* c, const int64_t* codes_dev, int32_t n_q, float* audio_out_dev,
                                void* stream);
/* Frames decoded since the last reset (= next transformer position).  Synchronises `stream`. */
int32_t vuib_codec_position(VuibCodec* c, int32_t* pos, void* stream);
/* Reads and clears the codec's device flag (code outside [0, 2048), position beyond max_seq: both are
 * clamped, never dereferenced).  Synchronises `stream`. */
int32_t vuib_codec_check_flag(VuibCodec* c, void* stream);
/* Intermediate activations of the last frame, for parity tests: which = 0 quantizer output (512),
 * 1 transformer output (1024), 2 upsampled latent (1024 x 4), 3 decoder.0 output (1536 x 4),
 * 4..7 output of decoder block 1..4 (C x T).  Copies n floats to out_host.  Synchronous. */
int32_t vuib_codec_read_tap(VuibCodec* c, int32_t which, float* out_host, int32_t n, void* stream);
int64_t vuib_codec_launch_count(VuibCodec* c);

/* ---------------------------------------------------------------------------
 * Codec encoder: 24 kHz audio -> 16 codebook indices per 80 ms frame, fp32.
 * Replaces the device work of QwenCodecEncoder.forward (src/vui/qwen_codec.py:385-390) as
 * StreamingCodecEncoder re-runs it over its fixed 10 s buffer on every feed()/flush() (671-805).
 * Weight pointers are borrowed and in torch's layouts.
 * ------------------------------------------------------------------------- */
typedef struct VuibCodecEncConfig {
    int32_t base_dim;        /* 64 */
    int32_t ratios[4];       /* 4, 5, 6, 8 */
    int32_t d_model;         /* 512 */
    int32_t n_layers;        /* 8 */
    int32_t n_heads;         /* 8 (x 64) */
    int32_t mlp_dim;         /* 2048 */
    int32_t max_samples;     /* 240000: the 10 s buffer; a multiple of 1920 */
} VuibCodecEncConfig;

typedef struct VuibEncResBlockW { VuibConvW c3; VuibConvW c1; } VuibEncResBlockW;   /* ResBlock, 278-290 */
typedef struct VuibEncLayerW {       /* EncTransformerBlock, 314-344 */
    const float *ln1_w, *ln1_b;
    const float* wqkv;     /* q_proj | k_proj | v_proj weights stacked by rows: (1536, 512) */
    const float *wo, *attn_scale, *ln2_w, *ln2_b, *fc1, *fc2, *mlp_scale;
} VuibEncLayerW;
typedef struct VuibCodecEncWeights {
    VuibConvW conv_in;               /* conv_encoder.layers.0: (64, 1, 7) */
    VuibEncResBlockW res[4];         /* layers.1, 4, 7, 10: (C/2, C, 3), (C, C/2, 1) */
    VuibConvW down[4];               /* layers.3, 6, 9, 12: (2C, C, 2r), stride r */
    VuibConvW conv_out;              /* layers.14: (512, 1024, 3) */
    VuibEncLayerW layer[VUIB_CODEC_LAYERS];
    const float* rope_cos;           /* (max_samples / 960, 64), RoPE.forward (161-171) */
    const float* rope_sin;
    const float* downsample;         /* downsample.conv.weight (512, 512, 4), stride 2, no bias */
    const float* sem_in;             /* quantizer.semantic.input_proj.weight (256, 512) */
    const float* acq_in;             /* quantizer.acoustic.input_proj.weight (256, 512) */
    const float* codebook[16];       /* semantic codebook 0, then acoustic 0..14: (2048, 256) */
    const float* codebook_norm2[16]; /* squared norm of every code: (2048) */
} VuibCodecEncWeights;

typedef struct VuibCodecEnc VuibCodecEnc;

int32_t vuib_codec_enc_create(const VuibCodecEncConfig* cfg, VuibCodecEnc** out);
int32_t vuib_codec_enc_destroy(VuibCodecEnc* c);
int32_t vuib_codec_enc_last_error(VuibCodecEnc* c, char* buf, size_t n);
int32_t vuib_codec_enc_workspace_bytes(VuibCodecEnc* c, size_t* bytes);
int32_t vuib_codec_enc_bind_workspace(VuibCodecEnc* c, void* dev, size_t bytes);
int32_t vuib_codec_enc_bind_weights(VuibCodecEnc* c, const VuibCodecEncWeights* w);
/* audio_dev float[n_samples] (n_samples a multiple of 1920, <= max_samples) -> codes_out_dev
 * int64[n_q][n_samples / 1920] (n_q <= 16).  Stateless: every call encodes from zero left padding. */
int32_t vuib_codec_enc_encode(VuibCodecEnc* c, const float* audio_dev, int32_t n_samples, int32_t n_q,
                              int64_t* codes_out_dev, void* stream);
/* Latents before quantisation of the last call, (512, n_samples / 1920) floats, for parity tests.  Synchronous. */
int32_t vuib_codec_enc_read_latent(VuibCodecEnc* c, float* out_host, int32_t n, void* stream);
int64_t vuib_codec_enc_launch_count(VuibCodecEnc* c);

#ifdef __cplusplus
}
#endif
#endif /* VUIB200_H */
