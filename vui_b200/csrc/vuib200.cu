// libvuib200: C ABI over the sm_100a decode kernels (see include/vuib200.h).
// Host side only validates, lays out the caller's workspace and enqueues
// kernels on the caller's stream; it never allocates device memory.
#include "../../include/vuib200.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <unordered_set>

#include "decode_kernels.cuh"
#include "tc_gemm.cuh"
#include "fused_blocks.cuh"
#include "depth_group.cuh"
#include "prefill_attn.cuh"

using namespace vuib;

struct WsLayout {
    size_t flag, ctl, row_slot, row_pos, x, q, attn, act, part, counters;
    size_t rq_x2, rq_x, rq_q, rq_act, rq_k, rq_v, rq_logits, code_cur;
    size_t frame_ctr, rep_counts, rep_hist, rep_head, rep_filled;
    size_t trace;
    size_t xn, rq_xn, rq_attn, tc_partial, tc_counters;
    size_t dg_layers, dg_head;   // box stream of the depth weights for k_depth_group (depth_group.cuh), 0 if none
    size_t fx_a, fx_b, fparts_a, fparts_b, rq_fx_a, rq_fx_b, rq_fparts_a, rq_fparts_b;
    size_t att_tiles, att_ntiles;
    size_t total;
};

constexpr int TC_PARTIAL_TILES = 224;  // most (tile, split) pairs of one GEMM launch
constexpr int FB_MLP_TH_BACKBONE = 512, FB_MLP_U_BACKBONE = 32;  // threads, hidden units per CTA of the MLP block
constexpr int FB_MLP_TH_DEPTH = 256, FB_MLP_U_DEPTH = 16;
constexpr int FUSED_MAX_PARTS = 16;     // most partial rows a fused block leaves (clusters of its grid)
constexpr int TRACE_STAMPS = 64;        // device-clock stamps kept for vuib_read_trace

// Tensor maps (TMA descriptors) of every weight matrix, built when the weights are bound.
struct TcMaps {
    CUtensorMap wqkv[VUIB_MAX_LAYERS], out_proj[VUIB_MAX_LAYERS], w1[VUIB_MAX_LAYERS], w3[VUIB_MAX_LAYERS],
        w2[VUIB_MAX_LAYERS];
    CUtensorMap rq_wqkv[VUIB_MAX_LAYERS], rq_out[VUIB_MAX_LAYERS], rq_w1[VUIB_MAX_LAYERS], rq_w3[VUIB_MAX_LAYERS],
        rq_w2[VUIB_MAX_LAYERS];
    CUtensorMap codec_head, rq_proj, rq_head;
    // un-swizzled maps whose box is one CTA's column slice of out_proj / w2 (fused single-row layers)
    CUtensorMap f_out[VUIB_MAX_LAYERS], f_w2[VUIB_MAX_LAYERS], f_rq_out[VUIB_MAX_LAYERS], f_rq_w2[VUIB_MAX_LAYERS];
    bool fused_backbone, fused_depth;
};

struct VuibEngine {
    VuibConfig cfg;
    VuibWeights w;
    bool have_w, have_kv, have_rope, have_ws;
    void* k[VUIB_MAX_LAYERS];
    void* v[VUIB_MAX_LAYERS];
    int32_t* seq_lens;
    const bf16* rope;
    unsigned char* ws;
    WsLayout lay;
    int R;        // rows of backbone scratch
    int S;        // attention splits per row
    VuibSampling samp;
    bf16* tap_layers;
    bf16* tap_rq;
    long long launches;
    int num_sms;        // 0 until a launch first asks the device
    unsigned spin_limit;  // bound of the waits inside kernels, in polls (vuib_set_wait_limit)
    int fused_backbone;   // 0 = not asked yet, 1 = the two-kernel layers can run here, -1 = they cannot
    int fused_depth;
    int depth_group;      // same for the one-launch depth loop of many streams
    bool dg_stream_ready; // the depth weights' box stream has been built in the workspace
    float* cb0_stats;   // optional (max_rows, 2) fp32: entropy and top probability of each cb0 draw
    TcMaps* tc;         // NULL until the weights are bound and the maps could be encoded
    struct HostFrame* host_frames;   // captured frames with host-side staging (vuib_frame_host_capture), a short list
    char err[256];
};

// One captured frame that starts and ends in pinned host memory: [staging -> codes_io] -> the frame's kernels ->
// [codes_io -> staging, eos_prob -> staging], as ONE graph launch.
struct HostFrame {
    int B;
    bool with_h2d;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    int64_t* stage_in;     // pinned (B, Q)
    int64_t* stage_out;    // pinned (B, Q)
    float* stage_eos;      // pinned (B)
    HostFrame* next;
};

static void free_host_frame(HostFrame* f) {
    if (f->exec) cudaGraphExecDestroy(f->exec);
    if (f->graph) cudaGraphDestroy(f->graph);
    if (f->stage_in) cudaFreeHost(f->stage_in);
    if (f->stage_out) cudaFreeHost(f->stage_out);
    if (f->stage_eos) cudaFreeHost(f->stage_eos);
    delete f;
}

static void free_host_frames(VuibEngine* e) {
    for (HostFrame* f = e->host_frames; f;) {
        HostFrame* n = f->next;
        free_host_frame(f);
        f = n;
    }
    e->host_frames = nullptr;
}

static int32_t fail(VuibEngine* e, int32_t code, const char* fmt, ...) {
    if (e) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(e->err, sizeof(e->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

static size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

static void make_layout(VuibEngine* e) {
    const VuibConfig& c = e->cfg;
    WsLayout& L = e->lay;
    const size_t R = e->R, RB = c.max_rows, d = c.d_model;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes); return o; };
    L.flag = take(256);
    L.ctl = take(sizeof(SamplingCtl));
    L.row_slot = take(R * 4);
    L.row_pos = take(R * 4);
    L.x = take(R * d * 2);
    L.q = take(R * (size_t)c.n_heads * HD * 2);
    L.attn = take(R * (size_t)c.n_heads * HD * 2);
    L.act = take(R * (size_t)c.ffn * 2);
    L.part = take(R * (size_t)c.n_heads * e->S * PART_STRIDE * 4);
    L.counters = take(R * (size_t)c.n_kv_heads * 4);
    const size_t rd = c.rq_d_model;
    L.rq_x2 = take(2 * RB * rd * 2);
    L.rq_x = take(RB * rd * 2);
    L.rq_q = take(2 * RB * rd * 2);
    L.rq_act = take(2 * RB * (size_t)c.rq_ffn * 2);
    L.rq_k = take((size_t)c.rq_n_layers * RB * c.n_quantizers * rd * 2);
    L.rq_v = take((size_t)c.rq_n_layers * RB * c.n_quantizers * rd * 2);
    L.rq_logits = take(RB * (size_t)c.codebook_size * 2);
    L.code_cur = take(RB * 4);
    L.frame_ctr = take((size_t)c.n_slots * 4);
    L.rep_counts = take((size_t)c.n_slots * c.codebook_size * 4);
    L.rep_hist = take((size_t)c.n_slots * REP_HIST_MAX * 4);
    L.rep_head = take((size_t)c.n_slots * 4);
    L.rep_filled = take((size_t)c.n_slots * 4);
    L.trace = take((size_t)TRACE_STAMPS * 8);
    L.xn = take(R * (size_t)(c.ffn > c.d_model ? c.ffn : c.d_model) * 2);
    L.rq_xn = take(2 * RB * rd * 2);
    L.rq_attn = take(2 * RB * rd * 2);
    L.tc_partial = take((size_t)(TC_PARTIAL_TILES + 80) * TC_TILE_N * (R < 256 ? ((R + 15) / 16) * 16 : 256) * 4);
    L.tc_counters = take(2 * 256 * 4);
    L.dg_layers = L.dg_head = 0;
    if (c.rq_d_model == DG_D && c.rq_n_heads == DG_CL && c.rq_n_layers <= DG_LAYERS && c.rq_ffn % DG_CL == 0 &&
        c.rq_ffn / DG_CL <= 192 && c.codebook_size == DG_CL * 256) {
        const int n_ub = (c.rq_ffn / DG_CL + 63) / 64;
        L.dg_layers = take((size_t)c.rq_n_layers * DG_CL * dg_boxes_per_layer(n_ub) * DG_BOX_BYTES);
        L.dg_head = take((size_t)(c.n_quantizers - 1) * DG_CL * 32 * DG_BOX_BYTES);
    }
    // fused two-kernel layers (single row): x as each block sees it, and the partial rows between blocks
    L.fx_a = take(d * 2);
    L.fx_b = take(d * 2);
    L.fparts_a = take((size_t)FUSED_MAX_PARTS * d * 4);
    L.fparts_b = take((size_t)FUSED_MAX_PARTS * d * 4);
    L.rq_fx_a = take(rd * 2);
    L.rq_fx_b = take(rd * 2);
    L.rq_fparts_a = take((size_t)FUSED_MAX_PARTS * rd * 4);
    L.rq_fparts_b = take((size_t)FUSED_MAX_PARTS * rd * 4);
    // query tiles of a prefill call (first row, rows) and their count
    L.att_tiles = take(2 * R * 4);
    L.att_ntiles = take(256);
    L.total = off;
}

// Launch with the programmatic-stream-serialization attribute (see pdl_wait in
// decode_kernels.cuh) unless VUIB_NO_PDL is set in the environment.
static bool env_off(const char* name) {
    const char* s = getenv(name);
    return s && s[0] && s[0] != '0';
}

static bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* s = getenv("VUIB_NO_PDL");
        v = (s && s[0] && s[0] != '0') ? 0 : 1;
    }
    return v == 1;
}

// Every kernel of a frame asks for the same (largest) shared-memory carve-out.  The tensor-core
// GEMM needs ~100-200 KB of shared memory and the small kernels between two GEMMs need almost
// none; left to their own preferences the SMs would re-partition L1/shared memory at every
// switch, which drains them and blocks the overlap of consecutive launches.
static void prefer_max_smem(const void* kern) {
    static std::mutex mu;
    static std::unordered_set<const void*> done;
    std::lock_guard<std::mutex> lock(mu);
    if (done.insert(kern).second)
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

template <class... KArgs, class... Args>
static cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                          Args... args) {
    prefer_max_smem(reinterpret_cast<const void*>(kern));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <class T>
static T* wsp(VuibEngine* e, size_t off) { return reinterpret_cast<T*>(e->ws + off); }

static void build_tc_maps(VuibEngine* e);
static int32_t build_dg_stream(VuibEngine* e);

// ---------------------------------------------------------------------------
// GEMV launch: pick the row-tile size from M, K from the supported set.
// ---------------------------------------------------------------------------
template <int K, class Stage, class Epi>
static cudaError_t launch_gemv_k(VuibEngine* e, const Stage& st, const Epi& ep, int M, int n_items,
                                 cudaStream_t s) {
    const int grid = (n_items + GEMV_WARPS - 1) / GEMV_WARPS;
    e->launches++;
    if (M <= 1) return launch(k_gemv<K, 1, Stage, Epi>, grid, GEMV_THREADS, 1 * K * 2, s, st, ep, M, n_items);
    if (M <= 2) return launch(k_gemv<K, 2, Stage, Epi>, grid, GEMV_THREADS, 2 * K * 2, s, st, ep, M, n_items);
    if (M <= 4) return launch(k_gemv<K, 4, Stage, Epi>, grid, GEMV_THREADS, 4 * K * 2, s, st, ep, M, n_items);
    return launch(k_gemv<K, 8, Stage, Epi>, grid, GEMV_THREADS, 8 * K * 2, s, st, ep, M, n_items);
}

#define VUIB_GEMV(Kval, ...)                                                        \
    [&]() -> cudaError_t {                                                          \
        switch (Kval) {                                                             \
            case 512: return launch_gemv_k<512>(__VA_ARGS__);                       \
            case 1024: return launch_gemv_k<1024>(__VA_ARGS__);                     \
            case 1408: return launch_gemv_k<1408>(__VA_ARGS__);                     \
            case 1536: return launch_gemv_k<1536>(__VA_ARGS__);                     \
            case 3072: return launch_gemv_k<3072>(__VA_ARGS__);                     \
            default: return cudaErrorInvalidValue;                                  \
        }                                                                           \
    }()

#define CK(call)                                                                              \
    do {                                                                                      \
        cudaError_t _err = (call);                                                            \
        if (_err != cudaSuccess)                                                              \
            return fail(e, VUIB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(_err));  \
    } while (0)

static bool k_supported(int K) {
    return K == 512 || K == 1024 || K == 1408 || K == 1536 || K == 3072;
}

// ---------------------------------------------------------------------------
// Handle lifecycle
// ---------------------------------------------------------------------------
extern "C" int32_t vuib_abi_version(void) { return VUIB_ABI_VERSION; }

extern "C" int32_t vuib_create(const VuibConfig* cfg, VuibEngine** out) {
    if (!cfg || !out) return VUIB_ERR_NULL;
    *out = nullptr;
    const VuibConfig& c = *cfg;
    const int G = c.n_kv_heads > 0 ? c.n_heads / c.n_kv_heads : 0;
    const bool ok = c.head_dim == HD && c.d_model == c.n_heads * HD && c.n_kv_heads > 0 &&
                    c.n_heads % c.n_kv_heads == 0 && (G == 1 || G == 2) &&
                    k_supported(c.d_model) && k_supported(c.ffn) && k_supported(c.rq_d_model) &&
                    k_supported(c.rq_ffn) && c.rq_d_model == c.rq_n_heads * HD &&
                    c.codebook_size == SAMPLE_THREADS * SAMPLE_EL && c.n_quantizers >= 2 &&
                    c.n_quantizers <= 16 && c.n_layers >= 1 && c.n_layers <= VUIB_MAX_LAYERS &&
                    c.rq_n_layers >= 1 && c.rq_n_layers <= VUIB_MAX_LAYERS;
    if (!ok) return VUIB_ERR_SHAPE;
    if (c.n_slots < 1 || c.max_seq < 1 || c.max_rows < 1 || c.max_prefill_rows < 1)
        return VUIB_ERR_RANGE;
    VuibEngine* e = new (std::nothrow) VuibEngine();
    if (!e) return VUIB_ERR_NULL;
    memset(e, 0, sizeof(*e));
    e->cfg = c;
    e->R = c.max_rows > c.max_prefill_rows ? c.max_rows : c.max_prefill_rows;
    e->S = (c.max_seq + ATT_SPLIT - 1) / ATT_SPLIT;
    e->samp.temperature = 1.0f;
    e->samp.top_k_cb0 = 1;
    e->samp.top_k_rq = 1;
    e->samp.rep_penalty = 1.0f;
    e->spin_limit = TC_SPIN_LIMIT;
    make_layout(e);
    *out = e;
    return VUIB_OK;
}

extern "C" int32_t vuib_destroy(VuibEngine* e) {
    if (e) {
        free_host_frames(e);
        delete e->tc;
    }
    delete e;
    return VUIB_OK;
}

extern "C" int32_t vuib_last_error(VuibEngine* e, char* buf, size_t n) {
    if (!e || !buf || n == 0) return VUIB_ERR_NULL;
    strncpy(buf, e->err, n - 1);
    buf[n - 1] = 0;
    return VUIB_OK;
}

extern "C" int64_t vuib_launch_count(VuibEngine* e) { return e ? e->launches : 0; }

extern "C" int32_t vuib_workspace_bytes(VuibEngine* e, size_t* bytes) {
    if (!e || !bytes) return VUIB_ERR_NULL;
    *bytes = e->lay.total;
    return VUIB_OK;
}

extern "C" int32_t vuib_bind_workspace(VuibEngine* e, void* dev, size_t bytes) {
    if (!e || !dev) return VUIB_ERR_NULL;
    if (bytes < e->lay.total || ((uintptr_t)dev & 255))
        return fail(e, VUIB_ERR_WORKSPACE, "workspace needs %zu bytes, 256-byte aligned; got %zu at %p",
                    e->lay.total, bytes, dev);
    e->ws = static_cast<unsigned char*>(dev);
    e->have_ws = true;
    return build_dg_stream(e);
}

extern "C" int32_t vuib_bind_weights(VuibEngine* e, const VuibWeights* w) {
    if (!e || !w) return VUIB_ERR_NULL;
    const VuibConfig& c = e->cfg;
    bool ok = w->audio_emb && w->codec_head && w->eos_w && w->eos_b && w->final_norm &&
              w->rq_backbone_proj && w->rq_code_emb && w->rq_pos_emb && w->rq_head && w->rq_norm;
    for (int i = 0; i < c.n_layers; ++i)
        ok = ok && w->attn_norm[i] && w->wqkv[i] && w->out_proj[i] && w->mlp_norm[i] && w->w1[i] &&
             w->w3[i] && w->w2[i];
    for (int i = 0; i < c.rq_n_layers; ++i)
        ok = ok && w->rq_attn_norm[i] && w->rq_wqkv[i] && w->rq_out_proj[i] && w->rq_mlp_norm[i] &&
             w->rq_w1[i] && w->rq_w3[i] && w->rq_w2[i];
    if (!ok) return fail(e, VUIB_ERR_NULL, "a weight pointer is NULL");
    e->w = *w;
    e->have_w = true;
    build_tc_maps(e);
    return build_dg_stream(e);
}

extern "C" int32_t vuib_bind_kv(VuibEngine* e, void* const* k_dev, void* const* v_dev,
                                int32_t* seq_lens_dev) {
    if (!e || !k_dev || !v_dev || !seq_lens_dev) return VUIB_ERR_NULL;
    for (int i = 0; i < e->cfg.n_layers; ++i) {
        if (!k_dev[i] || !v_dev[i]) return fail(e, VUIB_ERR_NULL, "KV pointer of layer %d is NULL", i);
        e->k[i] = k_dev[i];
        e->v[i] = v_dev[i];
    }
    e->seq_lens = seq_lens_dev;
    e->have_kv = true;
    return VUIB_OK;
}

extern "C" int32_t vuib_bind_rope(VuibEngine* e, const void* freqs_cis_dev) {
    if (!e || !freqs_cis_dev) return VUIB_ERR_NULL;
    e->rope = static_cast<const bf16*>(freqs_cis_dev);
    e->have_rope = true;
    return VUIB_OK;
}

static int32_t ready(VuibEngine* e) {
    if (!e) return VUIB_ERR_NULL;
    if (!(e->have_w && e->have_kv && e->have_rope && e->have_ws))
        return fail(e, VUIB_ERR_UNBOUND, "bind weights, kv, rope table and workspace first");
    return VUIB_OK;
}

extern "C" int32_t vuib_set_sampling(VuibEngine* e, const VuibSampling* s, void* stream) {
    if (!e || !s) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    if (!(s->temperature > 0.f)) return fail(e, VUIB_ERR_RANGE, "temperature must be > 0");
    if (s->n_codebooks < 0 || s->n_codebooks == 1 || s->n_codebooks > e->cfg.n_quantizers)
        return fail(e, VUIB_ERR_RANGE, "n_codebooks must be 0 or in [2, %d]", e->cfg.n_quantizers);
    if (s->rep_window < 0 || s->rep_window > REP_HIST_MAX)
        return fail(e, VUIB_ERR_RANGE, "rep_window must be in [0, %d]", REP_HIST_MAX);
    e->samp = *s;
    SamplingCtl ctl;
    ctl.temperature = s->temperature;
    ctl.top_k_cb0 = s->top_k_cb0;
    ctl.top_k_rq = s->top_k_rq;
    ctl.rep_penalty = s->rep_penalty;
    ctl.rep_window = s->rep_window;
    ctl.n_codebooks = s->n_codebooks;
    ctl.seed_lo = (uint32_t)(s->seed & 0xffffffffu);
    ctl.seed_hi = (uint32_t)(s->seed >> 32);
    CK(cudaMemcpyAsync(e->ws + e->lay.ctl, &ctl, sizeof(ctl), cudaMemcpyHostToDevice,
                       static_cast<cudaStream_t>(stream)));
    // the source is a stack object: make sure the copy has read it before returning
    CK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return VUIB_OK;
}

extern "C" int32_t vuib_set_stats(VuibEngine* e, float* cb0_stats_dev) {
    if (!e) return VUIB_ERR_NULL;
    e->cb0_stats = cb0_stats_dev;
    return VUIB_OK;
}

extern "C" int32_t vuib_set_taps(VuibEngine* e, void* layer_hidden_dev, void* rq_logits_dev) {
    if (!e) return VUIB_ERR_NULL;
    e->tap_layers = static_cast<bf16*>(layer_hidden_dev);
    e->tap_rq = static_cast<bf16*>(rq_logits_dev);
    return VUIB_OK;
}


// ---------------------------------------------------------------------------
// Tensor-core path (tc_gemm.cuh) for five rows and more: many streams, prefill.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D bf16 row-major (rows, cols) tensor, boxes of box_rows x 64 columns, 128-byte swizzle.
static bool make_map(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {TC_KCHUNK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D bf16 row-major (rows, cols) tensor, dense boxes of box_rows x box_cols, no swizzle.
static bool make_map_plain(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
                           uint32_t box_cols) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || box_rows > 256 || box_cols > 256) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static void build_tc_maps(VuibEngine* e) {
    delete e->tc;
    e->tc = nullptr;
    const VuibConfig& c = e->cfg;
    if (c.d_model % 128 || c.ffn % 64 || c.rq_d_model % 128 || c.rq_ffn % 64 || c.codebook_size % 128) return;
    TcMaps* t = new (std::nothrow) TcMaps();
    if (!t) return;
    bool ok = true;
    const int d = c.d_model, qkv = (c.n_heads + 2 * c.n_kv_heads) * HD, rd = c.rq_d_model;
    for (int i = 0; i < c.n_layers && ok; ++i) {
        ok = ok && make_map(&t->wqkv[i], e->w.wqkv[i], qkv, d, 64) && make_map(&t->out_proj[i], e->w.out_proj[i], d, d, 64) &&
             make_map(&t->w1[i], e->w.w1[i], c.ffn, d, 64) && make_map(&t->w3[i], e->w.w3[i], c.ffn, d, 64) &&
             make_map(&t->w2[i], e->w.w2[i], d, c.ffn, 64);
    }
    for (int i = 0; i < c.rq_n_layers && ok; ++i) {
        ok = ok && make_map(&t->rq_wqkv[i], e->w.rq_wqkv[i], 3 * rd, rd, 64) &&
             make_map(&t->rq_out[i], e->w.rq_out_proj[i], rd, rd, 64) &&
             make_map(&t->rq_w1[i], e->w.rq_w1[i], c.rq_ffn, rd, 64) &&
             make_map(&t->rq_w3[i], e->w.rq_w3[i], c.rq_ffn, rd, 64) &&
             make_map(&t->rq_w2[i], e->w.rq_w2[i], rd, c.rq_ffn, 64);
    }
    ok = ok && make_map(&t->codec_head, e->w.codec_head, c.codebook_size, d, 64) &&
         make_map(&t->rq_proj, e->w.rq_backbone_proj, rd, d, 64) &&
         make_map(&t->rq_head, e->w.rq_head, (uint64_t)(c.n_quantizers - 1) * c.codebook_size, rd, 64);
    if (!ok) {
        delete t;
        return;
    }
    // fused single-row layers: shapes checked again where they are used
    t->fused_backbone = c.d_model == 1024 && c.n_heads == 16 && c.n_kv_heads == 8 && c.ffn == 3072;
    for (int i = 0; i < c.n_layers && t->fused_backbone; ++i)
        t->fused_backbone = make_map_plain(&t->f_out[i], e->w.out_proj[i], d, d, d / FB_CL, 2 * HD) &&
                            make_map_plain(&t->f_w2[i], e->w.w2[i], d, c.ffn, d / FB_CL, FB_MLP_U_BACKBONE * FB_CL);
    t->fused_depth = rd == 512 && c.rq_n_heads == 8 && (c.rq_ffn == 1408 || c.rq_ffn == 1536);
    for (int i = 0; i < c.rq_n_layers && t->fused_depth; ++i)
        t->fused_depth = make_map_plain(&t->f_rq_out[i], e->w.rq_out_proj[i], rd, rd, rd / FB_CL, HD) &&
                         make_map_plain(&t->f_rq_w2[i], e->w.rq_w2[i], rd, c.rq_ffn, rd / FB_CL, FB_MLP_U_DEPTH * FB_CL);
    e->tc = t;
}

// Copies the depth weights into the box stream k_depth_group reads (once per binding; needs both the weights and
// the workspace).  Runs on the legacy default stream and waits for it: binding happens outside any capture.
static int32_t build_dg_stream(VuibEngine* e) {
    e->dg_stream_ready = false;
    if (!e->have_w || !e->have_ws || !e->lay.dg_layers) return VUIB_OK;
    const VuibConfig& c = e->cfg;
    DgStreamBuild b;
    memset(&b, 0, sizeof(b));
    for (int i = 0; i < c.rq_n_layers; ++i) {
        b.wqkv[i] = static_cast<const bf16*>(e->w.rq_wqkv[i]);
        b.out[i] = static_cast<const bf16*>(e->w.rq_out_proj[i]);
        b.w1[i] = static_cast<const bf16*>(e->w.rq_w1[i]);
        b.w3[i] = static_cast<const bf16*>(e->w.rq_w3[i]);
        b.w2[i] = static_cast<const bf16*>(e->w.rq_w2[i]);
    }
    b.head = static_cast<const bf16*>(e->w.rq_head);
    b.layers = e->ws + e->lay.dg_layers;
    b.head_out = e->ws + e->lay.dg_head;
    b.n_layers = c.rq_n_layers;
    b.ffn = c.rq_ffn;
    b.upc = c.rq_ffn / DG_CL;
    b.n_ub = (b.upc + 63) / 64;
    b.CS = c.codebook_size;
    b.n_head_pos = c.n_quantizers - 1;
    const int boxes = c.rq_n_layers * DG_CL * dg_boxes_per_layer(b.n_ub) + b.n_head_pos * DG_CL * 32;
    k_build_dg_stream<<<boxes, 256>>>(b);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(0));
    e->dg_stream_ready = true;
    return VUIB_OK;
}

static bool tc_ok(VuibEngine* e, int M) {
    // measured: 8 rows take 3.7 ms/frame on the register-tile GEMV, 16 rows 3.4 ms on the tensor cores
    return M > 4 && e->tc && !env_off("VUIB_NO_TC");
}

// D = W X^T over all M rows in blocks of <= 256, epilogue ep (see tc_gemm.cuh).
//  units: weight rows (N, multiple of 128) or, for the paired SwiGLU form, hidden units (multiple of 64).
template <class Epi>
static int32_t tc_gemm(VuibEngine* e, const CUtensorMap& a0, const CUtensorMap& a1, const bf16* X, int M, int K,
                       int units, int row_off, const Epi& ep, cudaStream_t s) {
    const WsLayout& L = e->lay;
    const int tiles = Epi::PAIRED ? units / 64 : units / TC_TILE_N;
    const int chunks_total = K / TC_KCHUNK;
    // Split K over enough CTAs to occupy the SMs (one MMA of this shape takes ~96 ns whatever the
    // batch, so the tensor pipe of ONE SM consumes weights at only ~42 GB/s).  The CTAs of a tile
    // meet on a counter, so the grid must be resident at once: at most two CTAs per SM.
    if (e->num_sms == 0) {
        int dev = 0;
        CK(cudaGetDevice(&dev));
        CK(cudaDeviceGetAttribute(&e->num_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    // Row blocks: up to 256 activation rows per CTA; a prefill of more rows is ONE launch whose grid's z
    // dimension walks the blocks (every weight tile is then read by its row blocks back to back and stays in
    // L2), not one launch per block.
    const int Mpad = M <= 256 ? (M + 15) / 16 * 16 : 256;
    const int m_blocks = (M + Mpad - 1) / Mpad;
    int splits = 1;
    for (int d = 2; d <= 16; d *= 2) {
        if (d > chunks_total || tiles * m_blocks * d > e->num_sms + e->num_sms / 2) break;
        if (Epi::PAIRED && d == 2) continue;
        splits = d;
    }
    const int max_smem = 202 * 1024;
    {   // a function attribute belongs to one device's copy of the kernel: set it once per device
        static std::mutex mu;
        static bool attr_set[64];
        int dev = 0;
        CK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            CK(cudaFuncSetAttribute(k_gemm_tc<Epi>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
            if (dev >= 0 && dev < 64) attr_set[dev] = true;
        }
    }
    CUtensorMap mx;
    if (!make_map(&mx, X, M, K, Mpad)) return fail(e, VUIB_ERR_CUDA, "cuTensorMapEncodeTiled failed");
    TcArgs ta;
    ta.N = units;
    ta.row_off = row_off;
    ta.M = M;
    ta.Mpad = Mpad;
    ta.chunks = chunks_total;
    ta.splits = splits;
    ta.tiles = tiles;
    ta.partial = wsp<float>(e, L.tc_partial);
    ta.counters = wsp<int32_t>(e, L.tc_counters);
    ta.flag = wsp<int32_t>(e, L.flag);
    ta.dbg = env_off("VUIB_TRACE") ? wsp<unsigned long long>(e, L.trace) : nullptr;
    ta.spin_limit = e->spin_limit;
    const int min_chunks = chunks_total / splits;  // the shortest split
    const size_t stage_bytes = TC_TILE_N * TC_KCHUNK * 2 + ((Mpad * TC_KCHUNK * 2 + 1023) & ~1023);
    const size_t epi_bytes = Epi::STAGED ? (size_t)Mpad * TC_EPI_BYTES_PER_M : 0;
    // two CTAs per SM when split (all CTAs of the grid must be resident), the whole SM otherwise
    const size_t budget = (splits > 1 ? 100 : 200) * 1024;
    int stages = epi_bytes + stage_bytes <= budget ? (int)((budget - epi_bytes) / stage_bytes) : 1;
    if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
    if (stages > min_chunks) stages = min_chunks;
    ta.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + epi_bytes + 1024;
    CK(launch(k_gemm_tc<Epi>, dim3(splits, tiles, m_blocks), TC_THREADS, smem, s, a0, a1, mx, ta, ep));
    e->launches++;
    return VUIB_OK;
}

static int32_t norm_rows(VuibEngine* e, const bf16* x, const void* w, float eps, bf16* out, int M, int K, int row_mul,
                         int row_add, cudaStream_t s) {
    CK(launch(k_rmsnorm_rows, M, 128, 0, s, x, static_cast<const bf16*>(w), eps, out, K, row_mul, row_add));
    e->launches++;
    return VUIB_OK;
}

static int32_t run_layers_tc(VuibEngine* e, int M, cudaStream_t s, bool prefill) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    bf16* x = wsp<bf16>(e, L.x);
    bf16* xn = wsp<bf16>(e, L.xn);
    bf16* q = wsp<bf16>(e, L.q);
    bf16* attn = wsp<bf16>(e, L.attn);
    bf16* act = wsp<bf16>(e, L.act);
    const int32_t* row_slot = wsp<int32_t>(e, L.row_slot);
    const int32_t* row_pos = wsp<int32_t>(e, L.row_pos);
    const int d = c.d_model, qc = c.n_heads * HD, kvc = c.n_kv_heads * HD;
    int32_t rc;
    for (int li = 0; li < c.n_layers; ++li) {
        if ((rc = norm_rows(e, x, e->w.attn_norm[li], c.norm_eps, xn, M, d, 1, 0, s))) return rc;
        TcEpiQkv eq{q, qc, kvc, static_cast<bf16*>(e->k[li]), static_cast<bf16*>(e->v[li]), row_slot, row_pos,
                    c.max_seq, e->rope, 1, 0, 0};
        if ((rc = tc_gemm(e, e->tc->wqkv[li], e->tc->wqkv[li], xn, M, d, qc + 2 * kvc, 0, eq, s))) return rc;

        if (prefill && !env_off("VUIB_NO_PREFILL_ATTN")) {
            // query tile x key tile on the tensor cores; the tiles were cut once for the call
            PrefillAttnArgs pa{q, static_cast<const bf16*>(e->k[li]), static_cast<const bf16*>(e->v[li]), row_slot, row_pos,
                               wsp<int32_t>(e, L.att_tiles), wsp<int32_t>(e, L.att_ntiles), attn, c.n_heads, c.n_kv_heads,
                               c.max_seq};
            const int bound = (M + PA_TILE - 1) / PA_TILE + c.n_slots;  // more tiles than this are looped over
            const int gx = bound < 4 * 148 ? bound : 4 * 148;
            if (c.n_heads == 2 * c.n_kv_heads) CK(launch(k_prefill_attn<2>, dim3(gx, c.n_kv_heads), 256, 0, s, pa));
            else CK(launch(k_prefill_attn<1>, dim3(gx, c.n_kv_heads), 128, 0, s, pa));
        } else {
            AttnArgs aa{q, static_cast<const bf16*>(e->k[li]), static_cast<const bf16*>(e->v[li]),
                        row_slot, row_pos, wsp<float>(e, L.part), wsp<int32_t>(e, L.counters), attn,
                        c.n_heads, c.n_kv_heads, c.max_seq, e->S, nullptr, c.n_slots, wsp<int32_t>(e, L.flag)};
            CK(launch(k_attn_decode, dim3(e->S, c.n_kv_heads, M), ATT_THREADS, 0, s, aa));
        }
        e->launches++;

        TcEpiResidual eo{x, d, nullptr};
        if ((rc = tc_gemm(e, e->tc->out_proj[li], e->tc->out_proj[li], attn, M, qc, d, 0, eo, s))) return rc;

        if ((rc = norm_rows(e, x, e->w.mlp_norm[li], c.norm_eps, xn, M, d, 1, 0, s))) return rc;
        TcEpiSwiGLU eg{act, c.ffn};
        if ((rc = tc_gemm(e, e->tc->w1[li], e->tc->w3[li], xn, M, d, c.ffn, 0, eg, s))) return rc;

        bf16* tap = (e->tap_layers && M <= c.max_rows) ? e->tap_layers + (size_t)li * c.max_rows * d : nullptr;
        TcEpiResidual ew{x, d, tap};
        if ((rc = tc_gemm(e, e->tc->w2[li], e->tc->w2[li], act, M, c.ffn, d, 0, ew, s))) return rc;
    }
    return VUIB_OK;
}

static int32_t run_heads_tc(VuibEngine* e, int B, const bf16* hidden, bf16* cb0, bf16* eos, cudaStream_t s) {
    const VuibConfig& c = e->cfg;
    TcEpiLogits el{cb0, c.codebook_size, nullptr, 0};
    int32_t rc = tc_gemm(e, e->tc->codec_head, e->tc->codec_head, hidden, B, c.d_model, c.codebook_size, 0, el, s);
    if (rc) return rc;
    CK(launch(k_eos_rows, (B + 3) / 4, 128, 0, s, hidden, static_cast<const bf16*>(e->w.eos_w),
              static_cast<const bf16*>(e->w.eos_b), eos, B, c.d_model));
    e->launches++;
    return VUIB_OK;
}

static int32_t rq_layers_tc(VuibEngine* e, int M, bf16* x, int rows_per_b, int pos_base, cudaStream_t s) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    const int rd = c.rq_d_model, Q = c.n_quantizers;
    bf16* q = wsp<bf16>(e, L.rq_q);
    bf16* act = wsp<bf16>(e, L.rq_act);
    bf16* xn = wsp<bf16>(e, L.rq_xn);
    bf16* attn = wsp<bf16>(e, L.rq_attn);
    const size_t layer_kv = (size_t)c.max_rows * Q * rd;
    int32_t rc;
    for (int li = 0; li < c.rq_n_layers; ++li) {
        bf16* kc = wsp<bf16>(e, L.rq_k) + li * layer_kv;
        bf16* vc = wsp<bf16>(e, L.rq_v) + li * layer_kv;
        if ((rc = norm_rows(e, x, e->w.rq_attn_norm[li], c.rq_norm_eps, xn, M, rd, 1, 0, s))) return rc;
        TcEpiQkv eq{q, rd, rd, kc, vc, nullptr, nullptr, Q, nullptr, rows_per_b, pos_base, 0};
        if ((rc = tc_gemm(e, e->tc->rq_wqkv[li], e->tc->rq_wqkv[li], xn, M, rd, 3 * rd, 0, eq, s))) return rc;

        StageRqAttn sa{q, kc, vc, c.rq_n_heads, Q, rows_per_b, pos_base};
        CK(launch(k_rq_attn_rows, M, 256, 0, s, sa, attn));
        e->launches++;

        TcEpiResidual eo{x, rd, nullptr};
        if ((rc = tc_gemm(e, e->tc->rq_out[li], e->tc->rq_out[li], attn, M, rd, rd, 0, eo, s))) return rc;

        if ((rc = norm_rows(e, x, e->w.rq_mlp_norm[li], c.rq_norm_eps, xn, M, rd, 1, 0, s))) return rc;
        TcEpiSwiGLU eg{act, c.rq_ffn};
        if ((rc = tc_gemm(e, e->tc->rq_w1[li], e->tc->rq_w3[li], xn, M, rd, c.rq_ffn, 0, eg, s))) return rc;

        TcEpiResidual ew{x, rd, nullptr};
        if ((rc = tc_gemm(e, e->tc->rq_w2[li], e->tc->rq_w2[li], act, M, c.rq_ffn, rd, 0, ew, s))) return rc;
    }
    return VUIB_OK;
}

// ---------------------------------------------------------------------------
// Single-row steps: each layer as two cluster kernels (fused_blocks.cuh).
// ---------------------------------------------------------------------------
// Where the residual stream is after a run of fused layers: x + bf16(sum of n_parts partial rows).
struct Residual {
    const bf16* x;
    const float* parts;
    int n_parts;
};

template <class... KArgs, class... Args>
static cudaError_t launch_cluster(void (*kern)(KArgs...), int n_clusters, int threads, size_t smem, cudaStream_t s,
                                  Args... args) {
    prefer_max_smem(reinterpret_cast<const void*>(kern));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_clusters * FB_CL);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FB_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Opts the kernel into its shared-memory size on the current device and asks whether `n_clusters`
// clusters of FB_CL CTAs can be resident at once.
template <class... KArgs>
static bool cluster_kernel_fits(void (*kern)(KArgs...), int n_clusters, int threads, size_t smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_clusters * FB_CL);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FB_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return n >= n_clusters;
}

static bool fused_backbone_ok(VuibEngine* e) {
    if (e->fused_backbone == 0) {
        const VuibConfig& c = e->cfg;
        bool ok = e->tc && e->tc->fused_backbone;
        ok = ok && cluster_kernel_fits(k_attn_block<1024, 2, false>, c.n_kv_heads, FB_THREADS, sizeof(AttnBlockSmem<1024, 2>));
        ok = ok && cluster_kernel_fits(k_mlp_block<1024, 3072, FB_MLP_U_BACKBONE, FB_MLP_TH_BACKBONE>,
                                       3072 / (FB_MLP_U_BACKBONE * FB_CL), FB_MLP_TH_BACKBONE,
                                       sizeof(MlpBlockSmem<1024, 3072, FB_MLP_U_BACKBONE, FB_MLP_TH_BACKBONE>));
        e->fused_backbone = ok ? 1 : -1;
    }
    return e->fused_backbone == 1 && !env_off("VUIB_NO_FUSED");
}

static bool fused_depth_ok(VuibEngine* e) {
    if (e->fused_depth == 0) {
        const VuibConfig& c = e->cfg;
        bool ok = e->tc && e->tc->fused_depth;
        ok = ok && cluster_kernel_fits(k_attn_block<512, 1, true>, c.rq_n_heads, FB_THREADS, sizeof(AttnBlockSmem<512, 1>));
        if (ok && c.rq_ffn == 1408)
            ok = cluster_kernel_fits(k_mlp_block<512, 1408, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>, 1408 / (FB_MLP_U_DEPTH * FB_CL),
                                     FB_MLP_TH_DEPTH, sizeof(MlpBlockSmem<512, 1408, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>));
        else if (ok)
            ok = cluster_kernel_fits(k_mlp_block<512, 1536, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>, 1536 / (FB_MLP_U_DEPTH * FB_CL),
                                     FB_MLP_TH_DEPTH, sizeof(MlpBlockSmem<512, 1536, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>));
        e->fused_depth = ok ? 1 : -1;
    }
    return e->fused_depth == 1 && !env_off("VUIB_NO_FUSED");
}

static PrefetchList prefetch_of(const void* a, size_t na, const void* b = nullptr, size_t nb = 0, const void* c = nullptr,
                                size_t nc = 0) {
    PrefetchList p;
    if (env_off("VUIB_NO_L2PF")) a = b = c = nullptr;
    p.ptr[0] = a; p.bytes[0] = na;
    p.ptr[1] = b; p.bytes[1] = nb;
    p.ptr[2] = c; p.bytes[2] = nc;
    return p;
}

// The backbone's blocks for ONE row whose (slot, position) is row 0 of the workspace table and whose
// input is L.x.  `after` names what follows the last block (its matrix is pulled into L2).
static int32_t run_layers_fused(VuibEngine* e, cudaStream_t s, Residual* out, const void* after, size_t after_bytes) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    const int d = c.d_model, qc = c.n_heads * HD, kvc = c.n_kv_heads * HD;
    const size_t qkv_bytes = (size_t)(qc + 2 * kvc) * d * 2, wo_bytes = (size_t)d * qc * 2;
    constexpr int NCL = 3072 / (FB_MLP_U_BACKBONE * FB_CL);
    bf16* xa = wsp<bf16>(e, L.fx_a);
    bf16* xb = wsp<bf16>(e, L.fx_b);
    float* pa = wsp<float>(e, L.fparts_a);
    float* pb = wsp<float>(e, L.fparts_b);
    for (int li = 0; li < c.n_layers; ++li) {
        AttnBlockArgs aa;
        memset(&aa, 0, sizeof(aa));
        aa.x_in = li == 0 ? wsp<bf16>(e, L.x) : xb;
        aa.parts_in = li == 0 ? nullptr : pb;
        aa.n_parts_in = li == 0 ? 0 : NCL;
        aa.x_out = xa;
        aa.tap = (e->tap_layers && li > 0) ? e->tap_layers + (size_t)(li - 1) * c.max_rows * d : nullptr;
        aa.norm_w = static_cast<const bf16*>(e->w.attn_norm[li]);
        aa.eps = c.norm_eps;
        aa.wqkv = static_cast<const bf16*>(e->w.wqkv[li]);
        aa.wo = static_cast<const bf16*>(e->w.out_proj[li]);
        aa.parts_out = pa;
        aa.k_cache = static_cast<bf16*>(e->k[li]);
        aa.v_cache = static_cast<bf16*>(e->v[li]);
        aa.row_slot = wsp<int32_t>(e, L.row_slot);
        aa.row_pos = wsp<int32_t>(e, L.row_pos);
        aa.max_seq = c.max_seq;
        aa.n_slots = c.n_slots;
        aa.rope = e->rope;
        aa.Hq = c.n_heads;
        aa.Hkv = c.n_kv_heads;
        aa.flag = wsp<int32_t>(e, L.flag);
        aa.spin_limit = e->spin_limit;
        // no L2 hint for the MLP block's matrices: that kernel is resident two launches ahead and copies them itself,
        // and 19 MB of hints during this block delayed its own loads (0.799 -> 0.788 ms per frame without them)
        aa.next = prefetch_of(nullptr, 0);
        if (env_off("VUIB_TRACE") && (li == 5 || li == 6)) aa.dbg = wsp<unsigned long long>(e, L.trace) + (li - 5) * 32;
        CK(launch_cluster(k_attn_block<1024, 2, false>, c.n_kv_heads, FB_THREADS, sizeof(AttnBlockSmem<1024, 2>), s, e->tc->f_out[li], aa));
        e->launches++;

        MlpBlockArgs ma;
        memset(&ma, 0, sizeof(ma));
        ma.x_in = xa;
        ma.parts_in = pa;
        ma.n_parts_in = c.n_kv_heads;
        ma.x_out = xb;
        ma.norm_w = static_cast<const bf16*>(e->w.mlp_norm[li]);
        ma.eps = c.norm_eps;
        ma.w1 = static_cast<const bf16*>(e->w.w1[li]);
        ma.w3 = static_cast<const bf16*>(e->w.w3[li]);
        ma.w2 = static_cast<const bf16*>(e->w.w2[li]);
        ma.parts_out = pb;
        if (li + 1 < c.n_layers && !env_off("VUIB_NO_KVHINT")) {
            ma.next_k = static_cast<const bf16*>(e->k[li + 1]);
            ma.next_v = static_cast<const bf16*>(e->v[li + 1]);
        }
        ma.row_slot = wsp<int32_t>(e, L.row_slot);
        ma.row_pos = wsp<int32_t>(e, L.row_pos);
        ma.max_seq = c.max_seq;
        ma.kvcols = kvc;
        ma.n_slots = c.n_slots;
        ma.flag = wsp<int32_t>(e, L.flag);
        ma.spin_limit = e->spin_limit;
        ma.next = li + 1 < c.n_layers ? prefetch_of(e->w.wqkv[li + 1], qkv_bytes, e->w.out_proj[li + 1], wo_bytes)
                                      : prefetch_of(after, after_bytes);
        if (env_off("VUIB_TRACE") && (li == 5 || li == 6)) ma.dbg = wsp<unsigned long long>(e, L.trace) + (li - 5) * 32 + 16;
        CK(launch_cluster(k_mlp_block<1024, 3072, FB_MLP_U_BACKBONE, FB_MLP_TH_BACKBONE>, NCL, FB_MLP_TH_BACKBONE,
                          sizeof(MlpBlockSmem<1024, 3072, FB_MLP_U_BACKBONE, FB_MLP_TH_BACKBONE>), s, e->tc->f_w2[li], ma));
        e->launches++;
    }
    out->x = xb;
    out->parts = pb;
    out->n_parts = NCL;
    return VUIB_OK;
}

// The depth transformer's blocks for ONE stream (row 0) at depth position `pos`, input token x.
static int32_t rq_layers_fused(VuibEngine* e, const bf16* x, int pos, cudaStream_t s, Residual* out, const void* after,
                               size_t after_bytes) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    const int rd = c.rq_d_model, Q = c.n_quantizers;
    const size_t qkv_bytes = (size_t)3 * rd * rd * 2, wo_bytes = (size_t)rd * rd * 2;
    const int ncl = c.rq_ffn / (FB_MLP_U_DEPTH * FB_CL);
    bf16* xa = wsp<bf16>(e, L.rq_fx_a);
    bf16* xb = wsp<bf16>(e, L.rq_fx_b);
    float* pa = wsp<float>(e, L.rq_fparts_a);
    float* pb = wsp<float>(e, L.rq_fparts_b);
    const size_t layer_kv = (size_t)c.max_rows * Q * rd;
    for (int li = 0; li < c.rq_n_layers; ++li) {
        AttnBlockArgs aa;
        memset(&aa, 0, sizeof(aa));
        aa.x_in = li == 0 ? x : xb;
        aa.parts_in = li == 0 ? nullptr : pb;
        aa.n_parts_in = li == 0 ? 0 : ncl;
        aa.x_out = xa;
        aa.norm_w = static_cast<const bf16*>(e->w.rq_attn_norm[li]);
        aa.eps = c.rq_norm_eps;
        aa.wqkv = static_cast<const bf16*>(e->w.rq_wqkv[li]);
        aa.wo = static_cast<const bf16*>(e->w.rq_out_proj[li]);
        aa.parts_out = pa;
        aa.k_cache = wsp<bf16>(e, L.rq_k) + li * layer_kv;
        aa.v_cache = wsp<bf16>(e, L.rq_v) + li * layer_kv;
        aa.fixed_slot = 0;
        aa.fixed_pos = pos;
        aa.max_seq = Q;
        aa.n_slots = c.max_rows;
        aa.Hq = c.rq_n_heads;
        aa.Hkv = c.rq_n_heads;
        aa.flag = wsp<int32_t>(e, L.flag);
        aa.spin_limit = e->spin_limit;
        aa.next = prefetch_of(nullptr, 0);   // as in the backbone: the MLP block copies its own matrices early enough
        if (env_off("VUIB_TRACE_DEPTH") && pos == 8 && (li == 1 || li == 2)) aa.dbg = wsp<unsigned long long>(e, L.trace) + (li - 1) * 32;
        CK(launch_cluster(k_attn_block<512, 1, true>, c.rq_n_heads, FB_THREADS, sizeof(AttnBlockSmem<512, 1>), s, e->tc->f_rq_out[li], aa));
        e->launches++;

        MlpBlockArgs ma;
        memset(&ma, 0, sizeof(ma));
        ma.x_in = xa;
        ma.parts_in = pa;
        ma.n_parts_in = c.rq_n_heads;
        ma.x_out = xb;
        ma.norm_w = static_cast<const bf16*>(e->w.rq_mlp_norm[li]);
        ma.eps = c.rq_norm_eps;
        ma.w1 = static_cast<const bf16*>(e->w.rq_w1[li]);
        ma.w3 = static_cast<const bf16*>(e->w.rq_w3[li]);
        ma.w2 = static_cast<const bf16*>(e->w.rq_w2[li]);
        ma.parts_out = pb;
        ma.flag = wsp<int32_t>(e, L.flag);
        ma.spin_limit = e->spin_limit;
        ma.next = li + 1 < c.rq_n_layers ? prefetch_of(e->w.rq_wqkv[li + 1], qkv_bytes, e->w.rq_out_proj[li + 1], wo_bytes)
                                         : prefetch_of(after, after_bytes);
        if (env_off("VUIB_TRACE_DEPTH") && pos == 8 && (li == 1 || li == 2)) ma.dbg = wsp<unsigned long long>(e, L.trace) + (li - 1) * 32 + 16;
        if (c.rq_ffn == 1408)
            CK(launch_cluster(k_mlp_block<512, 1408, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>, ncl, FB_MLP_TH_DEPTH,
                              sizeof(MlpBlockSmem<512, 1408, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>), s, e->tc->f_rq_w2[li], ma));
        else
            CK(launch_cluster(k_mlp_block<512, 1536, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>, ncl, FB_MLP_TH_DEPTH,
                              sizeof(MlpBlockSmem<512, 1536, FB_MLP_U_DEPTH, FB_MLP_TH_DEPTH>), s, e->tc->f_rq_w2[li], ma));
        e->launches++;
    }
    out->x = xb;
    out->parts = pb;
    out->n_parts = ncl;
    return VUIB_OK;
}

// ---------------------------------------------------------------------------
// Backbone: 24 blocks over M rows whose (slot, position) are in the workspace.
// ---------------------------------------------------------------------------
static int32_t run_layers(VuibEngine* e, int M, cudaStream_t s, Residual* out, bool prefill = false,
                          const void* after = nullptr, size_t after_bytes = 0) {
    out->x = wsp<bf16>(e, e->lay.x);
    out->parts = nullptr;
    out->n_parts = 0;
    if (M == 1 && fused_backbone_ok(e)) return run_layers_fused(e, s, out, after, after_bytes);
    if (tc_ok(e, M)) return run_layers_tc(e, M, s, prefill);
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    bf16* x = wsp<bf16>(e, L.x);
    bf16* q = wsp<bf16>(e, L.q);
    bf16* attn = wsp<bf16>(e, L.attn);
    bf16* act = wsp<bf16>(e, L.act);
    const int32_t* row_slot = wsp<int32_t>(e, L.row_slot);
    const int32_t* row_pos = wsp<int32_t>(e, L.row_pos);
    const int d = c.d_model, qc = c.n_heads * HD, kvc = c.n_kv_heads * HD;
    for (int li = 0; li < c.n_layers; ++li) {
        StageNorm sn{x, static_cast<const bf16*>(e->w.attn_norm[li]), c.norm_eps, 1, 0};
        EpiQkv eq{static_cast<const bf16*>(e->w.wqkv[li]), d, q, qc, kvc,
                  static_cast<bf16*>(e->k[li]), static_cast<bf16*>(e->v[li]),
                  row_slot, row_pos, c.max_seq, e->rope, 1, 0, env_off("VUIB_NO_KVHINT") ? 0 : 1};
        CK(VUIB_GEMV(d, e, sn, eq, M, (qc + 2 * kvc) / 2, s));

        AttnArgs aa{q, static_cast<const bf16*>(e->k[li]), static_cast<const bf16*>(e->v[li]),
                    row_slot, row_pos, wsp<float>(e, L.part), wsp<int32_t>(e, L.counters), attn,
                    c.n_heads, c.n_kv_heads, c.max_seq, e->S, nullptr, c.n_slots, wsp<int32_t>(e, L.flag)};
        CK(launch(k_attn_decode, dim3(e->S, c.n_kv_heads, M), ATT_THREADS, 0, s, aa));
        e->launches++;
        CK(cudaGetLastError());

        StageCopy sc{attn};
        EpiResidual eo{static_cast<const bf16*>(e->w.out_proj[li]), qc, x, d, nullptr};
        CK(VUIB_GEMV(qc, e, sc, eo, M, d, s));

        StageNorm sm{x, static_cast<const bf16*>(e->w.mlp_norm[li]), c.norm_eps, 1, 0};
        EpiSwiGLU eg{static_cast<const bf16*>(e->w.w1[li]), static_cast<const bf16*>(e->w.w3[li]), d,
                     act, c.ffn};
        CK(VUIB_GEMV(d, e, sm, eg, M, c.ffn, s));

        StageCopy sa{act};
        bf16* tap = (e->tap_layers && M <= c.max_rows)
                        ? e->tap_layers + (size_t)li * c.max_rows * d : nullptr;
        EpiResidual ew{static_cast<const bf16*>(e->w.w2[li]), c.ffn, x, d, tap};
        CK(VUIB_GEMV(c.ffn, e, sa, ew, M, d, s));
    }
    return VUIB_OK;
}

static int32_t run_heads(VuibEngine* e, int B, const bf16* hidden, bf16* cb0, bf16* eos,
                         cudaStream_t s) {
    if (tc_ok(e, B)) return run_heads_tc(e, B, hidden, cb0, eos, s);
    const VuibConfig& c = e->cfg;
    StageCopy sc{hidden};
    EpiLogits el{static_cast<const bf16*>(e->w.codec_head), c.d_model, c.codebook_size, cb0,
                 static_cast<const bf16*>(e->w.eos_w), static_cast<const bf16*>(e->w.eos_b), eos,
                 nullptr, 0};
    CK(VUIB_GEMV(c.d_model, e, sc, el, B, c.codebook_size + 1, s));
    return VUIB_OK;
}

extern "C" int32_t vuib_prefill(VuibEngine* e, int32_t n_rows, const int32_t* row_slot_dev,
                                const int32_t* row_pos_dev, const void* emb_dev,
                                void* hidden_out_dev, void* stream) {
    int32_t rc = ready(e);
    if (rc) return rc;
    if (!row_slot_dev || !row_pos_dev || !emb_dev || !hidden_out_dev) return VUIB_ERR_NULL;
    if (n_rows < 1 || n_rows > e->cfg.max_prefill_rows)
        return fail(e, VUIB_ERR_RANGE, "n_rows %d outside [1, %d]", n_rows, e->cfg.max_prefill_rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const WsLayout& L = e->lay;
    const int d = e->cfg.d_model;
    CK(launch(k_check_rows, (n_rows + 255) / 256, 256, 0, s, row_slot_dev, row_pos_dev, wsp<int32_t>(e, L.row_slot),
              wsp<int32_t>(e, L.row_pos), n_rows, e->cfg.n_slots, e->cfg.max_seq, wsp<int32_t>(e, L.flag)));
    e->launches++;
    CK(cudaMemcpyAsync(e->ws + L.x, emb_dev, (size_t)n_rows * d * 2, cudaMemcpyDeviceToDevice, s));
    Residual res;
    if (tc_ok(e, n_rows)) {
        CK(launch(k_prefill_tiles, 1, 256, (size_t)n_rows * 4, s, static_cast<const int32_t*>(wsp<int32_t>(e, L.row_slot)),
                  static_cast<const int32_t*>(wsp<int32_t>(e, L.row_pos)), n_rows, wsp<int32_t>(e, L.att_tiles),
                  wsp<int32_t>(e, L.att_ntiles)));
        e->launches++;
    }
    rc = run_layers(e, n_rows, s, &res, true);
    if (rc) return rc;
    CK(launch(k_final_norm, n_rows, 128, 0, s, res.x, static_cast<const bf16*>(e->w.final_norm),
                                        e->cfg.norm_eps, static_cast<bf16*>(hidden_out_dev), d,
                                        nullptr, nullptr, nullptr, 0, res.parts, res.n_parts, nullptr));
    e->launches++;
    CK(cudaGetLastError());
    return VUIB_OK;
}

extern "C" int32_t vuib_backbone_step(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                                      const int32_t* seq_inc_dev, const int64_t* codes_in_dev,
                                      void* hidden_out_dev, void* cb0_out_dev, void* eos_out_dev,
                                      void* stream) {
    int32_t rc = ready(e);
    if (rc) return rc;
    if (!slots_dev || !codes_in_dev || !hidden_out_dev || !cb0_out_dev || !eos_out_dev)
        return VUIB_ERR_NULL;
    if (B < 1 || B > e->cfg.max_rows)
        return fail(e, VUIB_ERR_RANGE, "B %d outside [1, %d]", B, e->cfg.max_rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    CK(launch(k_embed_codes, B, 128, 0, s, codes_in_dev, slots_dev, e->seq_lens,
                                    static_cast<const bf16*>(e->w.audio_emb), wsp<bf16>(e, L.x),
                                    wsp<int32_t>(e, L.row_slot), wsp<int32_t>(e, L.row_pos), c.d_model,
                                    c.n_quantizers, c.codebook_size, c.n_slots, c.max_seq,
                                    wsp<int32_t>(e, L.flag)));
    e->launches++;
    CK(cudaGetLastError());
    Residual res;
    rc = run_layers(e, B, s, &res, false, e->w.codec_head, (size_t)c.codebook_size * c.d_model * 2);
    if (rc) return rc;
    bf16* last_tap = (e->tap_layers && res.n_parts) ? e->tap_layers + (size_t)(c.n_layers - 1) * c.max_rows * c.d_model : nullptr;
    CK(launch(k_final_norm, B, 128, 0, s, res.x, static_cast<const bf16*>(e->w.final_norm),
                                   c.norm_eps, static_cast<bf16*>(hidden_out_dev), c.d_model,
                                   wsp<int32_t>(e, L.row_slot), seq_inc_dev, e->seq_lens, 1, res.parts, res.n_parts,
                                   last_tap));
    e->launches++;
    CK(cudaGetLastError());
    return run_heads(e, B, static_cast<const bf16*>(hidden_out_dev), static_cast<bf16*>(cb0_out_dev),
                     static_cast<bf16*>(eos_out_dev), s);
}

extern "C" int32_t vuib_heads(VuibEngine* e, int32_t B, const void* hidden_dev, void* cb0_out_dev,
                              void* eos_out_dev, void* stream) {
    int32_t rc = ready(e);
    if (rc) return rc;
    if (!hidden_dev || !cb0_out_dev || !eos_out_dev) return VUIB_ERR_NULL;
    if (B < 1 || B > e->cfg.max_rows)
        return fail(e, VUIB_ERR_RANGE, "B %d outside [1, %d]", B, e->cfg.max_rows);
    return run_heads(e, B, static_cast<const bf16*>(hidden_dev), static_cast<bf16*>(cb0_out_dev),
                     static_cast<bf16*>(eos_out_dev), static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Depth step
// ---------------------------------------------------------------------------
static int32_t rq_layers(VuibEngine* e, int M, bf16* x, int rows_per_b, int pos_base,
                         cudaStream_t s) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    const int rd = c.rq_d_model, Q = c.n_quantizers;
    bf16* q = wsp<bf16>(e, L.rq_q);
    bf16* act = wsp<bf16>(e, L.rq_act);
    const size_t layer_kv = (size_t)c.max_rows * Q * rd;
    for (int li = 0; li < c.rq_n_layers; ++li) {
        bf16* kc = wsp<bf16>(e, L.rq_k) + li * layer_kv;
        bf16* vc = wsp<bf16>(e, L.rq_v) + li * layer_kv;
        StageNorm sn{x, static_cast<const bf16*>(e->w.rq_attn_norm[li]), c.rq_norm_eps, 1, 0};
        EpiQkv eq{static_cast<const bf16*>(e->w.rq_wqkv[li]), rd, q, rd, rd, kc, vc,
                  nullptr, nullptr, Q, nullptr, rows_per_b, pos_base, 0};
        CK(VUIB_GEMV(rd, e, sn, eq, M, 3 * rd / 2, s));

        StageRqAttn sa{q, kc, vc, c.rq_n_heads, Q, rows_per_b, pos_base};
        EpiResidual eo{static_cast<const bf16*>(e->w.rq_out_proj[li]), rd, x, rd, nullptr};
        CK(VUIB_GEMV(rd, e, sa, eo, M, rd, s));

        StageNorm sm{x, static_cast<const bf16*>(e->w.rq_mlp_norm[li]), c.rq_norm_eps, 1, 0};
        EpiSwiGLU eg{static_cast<const bf16*>(e->w.rq_w1[li]), static_cast<const bf16*>(e->w.rq_w3[li]),
                     rd, act, c.rq_ffn};
        CK(VUIB_GEMV(rd, e, sm, eg, M, c.rq_ffn, s));

        StageCopy sc{act};
        EpiResidual ew{static_cast<const bf16*>(e->w.rq_w2[li]), c.rq_ffn, x, rd, nullptr};
        CK(VUIB_GEMV(c.rq_ffn, e, sc, ew, M, rd, s));
    }
    return VUIB_OK;
}

// ---------------------------------------------------------------------------
// Many streams: the whole depth loop as one launch (depth_group.cuh).
// ---------------------------------------------------------------------------
static bool depth_group_ok(VuibEngine* e) {
    if (e->depth_group == 0) {
        const VuibConfig& c = e->cfg;
        bool ok = e->tc && c.rq_d_model == DG_D && c.rq_n_heads == DG_CL && c.rq_n_layers <= DG_LAYERS &&
                  c.rq_ffn % DG_CL == 0 && c.rq_ffn / DG_CL <= 192 && c.codebook_size == DG_CL * 256;
        if (ok) {
            ok = cudaFuncSetAttribute(k_depth_group<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)sizeof(DepthGroupSmem<8>)) == cudaSuccess &&
                 cudaFuncSetAttribute(k_depth_group<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)sizeof(DepthGroupSmem<16>)) == cudaSuccess;
            if (!ok) cudaGetLastError();
        }
        e->depth_group = ok ? 1 : -1;
    }
    return e->depth_group == 1 && e->dg_stream_ready && !env_off("VUIB_NO_DEPTH_GROUP");
}

static int32_t launch_depth_group(VuibEngine* e, int B, const SampleArgs& sa_base, int Qn, cudaStream_t s) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    DepthGroupStream maps;
    maps.layers = e->ws + L.dg_layers;
    maps.head = e->ws + L.dg_head;
    maps.boxes_per_layer = dg_boxes_per_layer((c.rq_ffn / DG_CL + 63) / 64);
    DepthGroupArgs a;
    memset(&a, 0, sizeof(a));
    a.B = B;
    a.n_layers = c.rq_n_layers;
    a.Q = c.n_quantizers;
    a.Qn = Qn;
    a.CS = c.codebook_size;
    a.upc = c.rq_ffn / DG_CL;
    a.max_rows = c.max_rows;
    a.eps = c.rq_norm_eps;
    a.x2 = wsp<bf16>(e, L.rq_x2);
    a.x1 = wsp<bf16>(e, L.rq_x);
    a.kc = wsp<bf16>(e, L.rq_k);
    a.vc = wsp<bf16>(e, L.rq_v);
    for (int i = 0; i < c.rq_n_layers; ++i) {
        a.attn_norm[i] = static_cast<const bf16*>(e->w.rq_attn_norm[i]);
        a.mlp_norm[i] = static_cast<const bf16*>(e->w.rq_mlp_norm[i]);
    }
    a.final_norm = static_cast<const bf16*>(e->w.rq_norm);
    a.logits = wsp<bf16>(e, L.rq_logits);
    a.tap = e->tap_rq;
    a.sa = sa_base;
    a.flag = wsp<int32_t>(e, L.flag);
    a.spin_limit = e->spin_limit;
    a.dbg = env_off("VUIB_TRACE_DEPTH") ? wsp<unsigned long long>(e, L.trace) : nullptr;
    // groups of 8 streams while they fit the clusters that can be resident at once, else of 16
    const bool r8 = (B + 7) / 8 <= 15;
    const int groups = r8 ? (B + 7) / 8 : (B + 15) / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(groups * DG_CL);
    cfg.blockDim = dim3(DG_THREADS);
    cfg.dynamicSmemBytes = r8 ? sizeof(DepthGroupSmem<8>) : sizeof(DepthGroupSmem<16>);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = DG_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    prefer_max_smem(reinterpret_cast<const void*>(r8 ? k_depth_group<8> : k_depth_group<16>));
    if (r8) CK(cudaLaunchKernelEx(&cfg, k_depth_group<8>, maps, a));
    else CK(cudaLaunchKernelEx(&cfg, k_depth_group<16>, maps, a));
    e->launches++;
    return VUIB_OK;
}

static int32_t run_depth(VuibEngine* e, int B, const int32_t* slots, const bf16* hidden,
                         const bf16* cb0_logits, const bf16* eos_logit, int first_frame,
                         int64_t* codes_out, float* eos_prob, cudaStream_t s) {
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    const int Q = c.n_quantizers, CS = c.codebook_size, rd = c.rq_d_model;
    const int Qn = e->samp.n_codebooks > 0 ? e->samp.n_codebooks : Q;
    int32_t* code_cur = wsp<int32_t>(e, L.code_cur);
    SampleArgs sa;
    memset(&sa, 0, sizeof(sa));
    sa.ctl = wsp<SamplingCtl>(e, L.ctl);
    sa.slots = slots;
    sa.frame_ctr = wsp<int32_t>(e, L.frame_ctr);
    sa.rep_counts = wsp<float>(e, L.rep_counts);
    sa.rep_hist = wsp<int32_t>(e, L.rep_hist);
    sa.rep_head = wsp<int32_t>(e, L.rep_head);
    sa.rep_filled = wsp<int32_t>(e, L.rep_filled);
    sa.code_cur = code_cur;
    sa.codes_out = codes_out;
    sa.Q = Q;
    sa.n_slots = c.n_slots;
    sa.flag = wsp<int32_t>(e, L.flag);

    // cb0
    sa.logits = cb0_logits;
    sa.stride = CS;
    sa.codebook = 0;
    sa.out_col = 0;
    sa.first_frame = first_frame;
    sa.eos_logit = eos_logit;
    sa.eos_prob = eos_prob;
    sa.bump_frame = 0;
    sa.zero_from = Qn < Q ? Qn : 0;
    sa.stats_out = e->cb0_stats;
    // the sampler also builds depth position 1 from the code it drew (rows 2b+1)
    sa.emb_out = wsp<bf16>(e, L.rq_x2);
    sa.code_emb = static_cast<const bf16*>(e->w.rq_code_emb);
    sa.pos_emb = static_cast<const bf16*>(e->w.rq_pos_emb);
    sa.emb_p = 1;
    sa.emb_rd = rd;
    sa.emb_row_mul = 2;
    sa.emb_row_add = 1;
    CK(launch(k_sample, B, SAMPLE_THREADS, 0, s, sa));
    e->launches++;
    CK(cudaGetLastError());
    sa.eos_logit = nullptr;
    sa.eos_prob = nullptr;
    sa.first_frame = 0;
    sa.zero_from = 0;

    // depth positions 0 (projected hidden) and 1 (code 0): rows 2b, 2b+1
    bf16* x2 = wsp<bf16>(e, L.rq_x2);
    bf16* x1 = wsp<bf16>(e, L.rq_x);
    const bf16* pos_emb = static_cast<const bf16*>(e->w.rq_pos_emb);
    const bool tc = tc_ok(e, B);
    int32_t rc;
    if (tc) {
        TcEpiProjPos ep{pos_emb, x2, rd, 2};
        if ((rc = tc_gemm(e, e->tc->rq_proj, e->tc->rq_proj, hidden, B, c.d_model, rd, 0, ep, s))) return rc;
    } else {
        StageCopy sc{hidden};
        EpiProjPos ep{static_cast<const bf16*>(e->w.rq_backbone_proj), c.d_model, pos_emb, x2, rd, 2};
        CK(VUIB_GEMV(c.d_model, e, sc, ep, B, rd, s));
    }
    if (tc && depth_group_ok(e)) return launch_depth_group(e, B, sa, Qn, s);
    rc = tc ? rq_layers_tc(e, 2 * B, x2, 2, 0, s) : rq_layers(e, 2 * B, x2, 2, 0, s);
    if (rc) return rc;

    bf16* logits = wsp<bf16>(e, L.rq_logits);
    const bf16* head = static_cast<const bf16*>(e->w.rq_head);
    const bool fused = B == 1 && fused_depth_ok(e);
    for (int i = 0; i < Qn - 1; ++i) {
        Residual res{i == 0 ? x2 : x1, nullptr, 0};
        if (i > 0) {
            if (fused) rc = rq_layers_fused(e, x1, i + 1, s, &res, head + (size_t)i * CS * rd, (size_t)CS * rd * 2);
            else rc = tc ? rq_layers_tc(e, B, x1, 1, i + 1, s) : rq_layers(e, B, x1, 1, i + 1, s);
            if (rc) return rc;
        }
        if (tc) {
            bf16* xn = wsp<bf16>(e, L.rq_xn);
            if ((rc = norm_rows(e, i == 0 ? x2 : x1, e->w.rq_norm, c.rq_norm_eps, xn, B, rd, i == 0 ? 2 : 1,
                                i == 0 ? 1 : 0, s)))
                return rc;
            TcEpiLogits el{logits, CS, e->tap_rq ? e->tap_rq + (size_t)i * CS : nullptr, (Q - 1) * CS};
            if ((rc = tc_gemm(e, e->tc->rq_head, e->tc->rq_head, xn, B, rd, CS, i * CS, el, s))) return rc;
        } else {
            StageNorm sn{res.x, static_cast<const bf16*>(e->w.rq_norm), c.rq_norm_eps,
                         i == 0 ? 2 : 1, i == 0 ? 1 : 0, res.parts, res.n_parts};
            EpiLogits el{head + (size_t)i * CS * rd, rd, CS, logits, nullptr, nullptr, nullptr,
                         e->tap_rq ? e->tap_rq + (size_t)i * CS : nullptr, (Q - 1) * CS};
            CK(VUIB_GEMV(rd, e, sn, el, B, CS, s));
        }
        sa.logits = logits;
        sa.codebook = i + 1;
        sa.out_col = i + 1;
        sa.bump_frame = (i == Qn - 2);
        sa.emb_out = (i + 1 < Qn - 1) ? x1 : nullptr;  // token of depth position i+2 for the next codebook
        sa.emb_p = i + 2;
        sa.emb_row_mul = 1;
        sa.emb_row_add = 0;
        CK(launch(k_sample, B, SAMPLE_THREADS, 0, s, sa));
        e->launches++;
        CK(cudaGetLastError());
    }
    return VUIB_OK;
}

extern "C" int32_t vuib_depth_step(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                                   const void* hidden_dev, const void* cb0_logits_dev,
                                   const void* eos_logit_dev, int32_t first_frame,
                                   int64_t* codes_out_dev, float* eos_prob_out_dev, void* stream) {
    int32_t rc = ready(e);
    if (rc) return rc;
    if (!slots_dev || !hidden_dev || !cb0_logits_dev || !codes_out_dev) return VUIB_ERR_NULL;
    if (B < 1 || B > e->cfg.max_rows)
        return fail(e, VUIB_ERR_RANGE, "B %d outside [1, %d]", B, e->cfg.max_rows);
    return run_depth(e, B, slots_dev, static_cast<const bf16*>(hidden_dev),
                     static_cast<const bf16*>(cb0_logits_dev), static_cast<const bf16*>(eos_logit_dev),
                     first_frame, codes_out_dev, eos_prob_out_dev, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t vuib_decode_frame(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                                     const int32_t* seq_inc_dev, int64_t* codes_io_dev,
                                     void* hidden_out_dev, void* cb0_out_dev, void* eos_out_dev,
                                     float* eos_prob_out_dev, void* stream) {
    int32_t rc = ready(e);
    if (rc) return rc;
    if (!slots_dev || !codes_io_dev || !hidden_out_dev || !cb0_out_dev || !eos_out_dev) return VUIB_ERR_NULL;
    if (B < 1 || B > e->cfg.max_rows)
        return fail(e, VUIB_ERR_RANGE, "B %d outside [1, %d]", B, e->cfg.max_rows);
    rc = vuib_backbone_step(e, B, slots_dev, seq_inc_dev, codes_io_dev, hidden_out_dev,
                            cb0_out_dev, eos_out_dev, stream);
    if (rc) return rc;
    return run_depth(e, B, slots_dev, static_cast<const bf16*>(hidden_out_dev),
                     static_cast<const bf16*>(cb0_out_dev), static_cast<const bf16*>(eos_out_dev), 0,
                     codes_io_dev, eos_prob_out_dev, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// A frame from and to host memory: what a serving loop does per codec frame, as one graph launch.
// ---------------------------------------------------------------------------
extern "C" int32_t vuib_frame_host_capture(VuibEngine* e, int32_t B, int32_t with_h2d, const int32_t* slots_dev,
                                           const int32_t* seq_inc_dev, int64_t* codes_io_dev, void* hidden_out_dev,
                                           void* cb0_out_dev, void* eos_out_dev, float* eos_prob_out_dev,
                                           void* stream) {
    int32_t rc = ready(e);
    if (rc) return rc;
    if (!slots_dev || !codes_io_dev || !hidden_out_dev || !cb0_out_dev || !eos_out_dev || !eos_prob_out_dev)
        return VUIB_ERR_NULL;
    if (B < 1 || B > e->cfg.max_rows) return fail(e, VUIB_ERR_RANGE, "B %d outside [1, %d]", B, e->cfg.max_rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!s) return fail(e, VUIB_ERR_RANGE, "capture needs a stream of its own, not the default stream");
    // a frame captured earlier for the same (B, with_h2d) is replaced
    for (HostFrame** pf = &e->host_frames; *pf; pf = &(*pf)->next)
        if ((*pf)->B == B && (*pf)->with_h2d == (with_h2d != 0)) {
            HostFrame* old = *pf;
            *pf = old->next;
            free_host_frame(old);
            break;
        }
    HostFrame* f = new (std::nothrow) HostFrame();
    if (!f) return fail(e, VUIB_ERR_CUDA, "out of host memory");
    memset(f, 0, sizeof(*f));
    f->B = B;
    f->with_h2d = with_h2d != 0;
    f->next = e->host_frames;
    e->host_frames = f;   // owned from here on: freed with the engine whatever happens below
    const size_t code_bytes = (size_t)B * e->cfg.n_quantizers * sizeof(int64_t);
    CK(cudaHostAlloc(reinterpret_cast<void**>(&f->stage_in), code_bytes, cudaHostAllocDefault));
    CK(cudaHostAlloc(reinterpret_cast<void**>(&f->stage_out), code_bytes, cudaHostAllocDefault));
    CK(cudaHostAlloc(reinterpret_cast<void**>(&f->stage_eos), (size_t)B * sizeof(float), cudaHostAllocDefault));
    memset(f->stage_in, 0, code_bytes);
    CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    cudaError_t ce = cudaSuccess;
    if (f->with_h2d) ce = cudaMemcpyAsync(codes_io_dev, f->stage_in, code_bytes, cudaMemcpyHostToDevice, s);
    rc = ce == cudaSuccess ? vuib_decode_frame(e, B, slots_dev, seq_inc_dev, codes_io_dev, hidden_out_dev, cb0_out_dev,
                                               eos_out_dev, eos_prob_out_dev, stream)
                           : VUIB_ERR_CUDA;
    if (rc == VUIB_OK) {
        ce = cudaMemcpyAsync(f->stage_out, codes_io_dev, code_bytes, cudaMemcpyDeviceToHost, s);
        if (ce == cudaSuccess)
            ce = cudaMemcpyAsync(f->stage_eos, eos_prob_out_dev, (size_t)B * sizeof(float), cudaMemcpyDeviceToHost, s);
    }
    cudaGraph_t g = nullptr;
    const cudaError_t end = cudaStreamEndCapture(s, &g);   // always ends the capture, also after a failure above
    f->graph = g;
    if (rc != VUIB_OK) return rc;
    if (ce != cudaSuccess) return fail(e, VUIB_ERR_CUDA, "capture: %s", cudaGetErrorString(ce));
    if (end != cudaSuccess || !g) return fail(e, VUIB_ERR_CUDA, "capture: %s", cudaGetErrorString(end));
    CK(cudaGraphInstantiate(&f->exec, f->graph, 0));
    return VUIB_OK;
}

extern "C" int32_t vuib_frame_host(VuibEngine* e, int32_t B, int32_t with_h2d, const int64_t* codes_in_host,
                                   int64_t* codes_out_host, float* eos_prob_out_host, void* stream) {
    if (!e || !codes_out_host) return VUIB_ERR_NULL;
    HostFrame* f = e->host_frames;
    while (f && !(f->B == B && f->with_h2d == (with_h2d != 0) && f->exec)) f = f->next;
    if (!f) return fail(e, VUIB_ERR_UNBOUND, "no captured frame for B = %d: call vuib_frame_host_capture first", B);
    if (f->with_h2d && !codes_in_host) return VUIB_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t code_bytes = (size_t)B * e->cfg.n_quantizers * sizeof(int64_t);
    if (f->with_h2d) memcpy(f->stage_in, codes_in_host, code_bytes);
    CK(cudaGraphLaunch(f->exec, s));
    CK(cudaStreamSynchronize(s));
    memcpy(codes_out_host, f->stage_out, code_bytes);
    if (eos_prob_out_host) memcpy(eos_prob_out_host, f->stage_eos, (size_t)B * sizeof(float));
    return VUIB_OK;
}

extern "C" int32_t vuib_attention(VuibEngine* e, int32_t layer, int32_t n_rows, const void* q_dev,
                                  const int32_t* row_slot_dev, const int32_t* row_pos_dev,
                                  void* out_dev, void* stream) {
    if (!e || !q_dev || !row_slot_dev || !row_pos_dev || !out_dev) return VUIB_ERR_NULL;
    if (!e->have_kv || !e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind kv and workspace first");
    const VuibConfig& c = e->cfg;
    if (layer < 0 || layer >= c.n_layers) return fail(e, VUIB_ERR_RANGE, "layer %d out of range", layer);
    if (n_rows < 1 || n_rows > e->R) return fail(e, VUIB_ERR_RANGE, "n_rows %d outside [1, %d]", n_rows, e->R);
    AttnArgs aa{static_cast<const bf16*>(q_dev), static_cast<const bf16*>(e->k[layer]),
                static_cast<const bf16*>(e->v[layer]), row_slot_dev, row_pos_dev,
                wsp<float>(e, e->lay.part), wsp<int32_t>(e, e->lay.counters), static_cast<bf16*>(out_dev),
                c.n_heads, c.n_kv_heads, c.max_seq, e->S, nullptr, c.n_slots, wsp<int32_t>(e, e->lay.flag)};
    CK(launch(k_attn_decode, dim3(e->S, c.n_kv_heads, n_rows), ATT_THREADS, 0, static_cast<cudaStream_t>(stream), aa));
    e->launches++;
    CK(cudaGetLastError());
    return VUIB_OK;
}

extern "C" int32_t vuib_embed_codes(VuibEngine* e, int32_t n_rows, const int64_t* codes_dev,
                                    void* out_dev, void* stream) {
    if (!e || !codes_dev || !out_dev) return VUIB_ERR_NULL;
    if (!e->have_w || !e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind weights and workspace first");
    if (n_rows < 1) return fail(e, VUIB_ERR_RANGE, "n_rows %d < 1", n_rows);
    const VuibConfig& c = e->cfg;
    CK(launch(k_embed_codes, n_rows, 128, 0, static_cast<cudaStream_t>(stream), 
        codes_dev, nullptr, nullptr, static_cast<const bf16*>(e->w.audio_emb), static_cast<bf16*>(out_dev),
        nullptr, nullptr, c.d_model, c.n_quantizers, c.codebook_size, c.n_slots, c.max_seq,
        wsp<int32_t>(e, e->lay.flag)));
    e->launches++;
    CK(cudaGetLastError());
    return VUIB_OK;
}

extern "C" int32_t vuib_sample_rows(VuibEngine* e, int32_t B, const int32_t* slots_dev,
                                    const void* logits_dev, int32_t codebook, int64_t* codes_out_dev,
                                    void* stream) {
    if (!e || !slots_dev || !logits_dev || !codes_out_dev) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    if (B < 1 || B > e->cfg.max_rows) return fail(e, VUIB_ERR_RANGE, "B %d outside [1, %d]", B, e->cfg.max_rows);
    if (codebook < 0 || codebook >= e->cfg.n_quantizers) return fail(e, VUIB_ERR_RANGE, "codebook %d", codebook);
    const WsLayout& L = e->lay;
    SampleArgs sa;
    memset(&sa, 0, sizeof(sa));
    sa.logits = static_cast<const bf16*>(logits_dev);
    sa.stride = e->cfg.codebook_size;
    sa.ctl = wsp<SamplingCtl>(e, L.ctl);
    sa.slots = slots_dev;
    sa.frame_ctr = wsp<int32_t>(e, L.frame_ctr);
    sa.codebook = codebook;
    sa.rep_counts = wsp<float>(e, L.rep_counts);
    sa.rep_hist = wsp<int32_t>(e, L.rep_hist);
    sa.rep_head = wsp<int32_t>(e, L.rep_head);
    sa.rep_filled = wsp<int32_t>(e, L.rep_filled);
    sa.code_cur = wsp<int32_t>(e, L.code_cur);
    sa.codes_out = codes_out_dev;
    sa.Q = 1;
    sa.out_col = 0;
    sa.bump_frame = 1;
    sa.n_slots = e->cfg.n_slots;
    sa.flag = wsp<int32_t>(e, L.flag);
    CK(launch(k_sample, B, SAMPLE_THREADS, 0, static_cast<cudaStream_t>(stream), sa));
    e->launches++;
    CK(cudaGetLastError());
    return VUIB_OK;
}

// ---------------------------------------------------------------------------
// Single fused ops on caller-supplied rows, for the parity tests: with an identity
// matrix as W the GEMV passes its staged input through exactly, so the RMSNorm
// staging and the RoPE epilogue can be held bit for bit against the reference's
// own module outputs.
// ---------------------------------------------------------------------------
extern "C" int32_t vuib_debug_norm_linear(VuibEngine* e, int32_t n_rows, const void* x_dev,
                                          const void* norm_w_dev, const void* w_dev, int32_t n_out,
                                          void* out_dev, int32_t tensor_cores, void* stream) {
    if (!e || !x_dev || !norm_w_dev || !w_dev || !out_dev) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    const VuibConfig& c = e->cfg;
    if (n_rows < 1 || n_rows > e->R || n_out < 1) return fail(e, VUIB_ERR_RANGE, "n_rows %d / n_out %d out of range", n_rows, n_out);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bf16* x = static_cast<const bf16*>(x_dev);
    const int d = c.d_model;
    if (tensor_cores) {
        if (n_out % TC_TILE_N) return fail(e, VUIB_ERR_RANGE, "n_out must be a multiple of %d on the tensor-core path", TC_TILE_N);
        CUtensorMap mw;
        if (!make_map(&mw, w_dev, n_out, d, 64)) return fail(e, VUIB_ERR_CUDA, "cuTensorMapEncodeTiled failed");
        bf16* xn = wsp<bf16>(e, e->lay.xn);
        int32_t rc = norm_rows(e, x, norm_w_dev, c.norm_eps, xn, n_rows, d, 1, 0, s);
        if (rc) return rc;
        TcEpiLogits el{static_cast<bf16*>(out_dev), n_out, nullptr, 0};
        return tc_gemm(e, mw, mw, xn, n_rows, d, n_out, 0, el, s);
    }
    StageNorm sn{x, static_cast<const bf16*>(norm_w_dev), c.norm_eps, 1, 0};
    EpiLogits el{static_cast<const bf16*>(w_dev), d, n_out, static_cast<bf16*>(out_dev), nullptr, nullptr, nullptr,
                 nullptr, 0};
    CK(VUIB_GEMV(d, e, sn, el, n_rows, n_out, s));
    return VUIB_OK;
}

extern "C" int32_t vuib_debug_linear_rope(VuibEngine* e, int32_t n_rows, const void* x_dev, const void* w_dev,
                                          const int32_t* row_pos_dev, void* out_dev, int32_t tensor_cores,
                                          void* stream) {
    if (!e || !x_dev || !w_dev || !row_pos_dev || !out_dev) return VUIB_ERR_NULL;
    if (!e->have_ws || !e->have_rope) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace and the rope table first");
    const VuibConfig& c = e->cfg;
    if (n_rows < 1 || n_rows > e->R) return fail(e, VUIB_ERR_RANGE, "n_rows %d outside [1, %d]", n_rows, e->R);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int d = c.d_model;
    // every output column is a "q" column: rotated at row_pos[r], nothing goes to a cache
    int32_t* row_slot = wsp<int32_t>(e, e->lay.row_slot);
    int32_t* row_pos = wsp<int32_t>(e, e->lay.row_pos);
    CK(cudaMemsetAsync(row_slot, 0, (size_t)n_rows * 4, s));
    CK(launch(k_check_rows, (n_rows + 255) / 256, 256, 0, s, static_cast<const int32_t*>(row_slot), row_pos_dev, row_slot,
              row_pos, n_rows, c.n_slots, c.max_seq, wsp<int32_t>(e, e->lay.flag)));
    e->launches++;
    if (tensor_cores) {
        CUtensorMap mw;
        if (!make_map(&mw, w_dev, d, d, 64)) return fail(e, VUIB_ERR_CUDA, "cuTensorMapEncodeTiled failed");
        TcEpiQkv eq{static_cast<bf16*>(out_dev), d, 0, nullptr, nullptr, row_slot, row_pos, c.max_seq, e->rope, 1, 0, 0};
        return tc_gemm(e, mw, mw, static_cast<const bf16*>(x_dev), n_rows, d, d, 0, eq, s);
    }
    StageCopy sc{static_cast<const bf16*>(x_dev)};
    EpiQkv eq{static_cast<const bf16*>(w_dev), d, static_cast<bf16*>(out_dev), d, 0, nullptr, nullptr,
              row_slot, row_pos, c.max_seq, e->rope, 1, 0, 0};
    CK(VUIB_GEMV(d, e, sc, eq, n_rows, d / 2, s));
    return VUIB_OK;
}

extern "C" int32_t vuib_rep_reset(VuibEngine* e, int32_t slot, void* stream) {
    if (!e) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    const VuibConfig& c = e->cfg;
    if (slot < -1 || slot >= c.n_slots) return fail(e, VUIB_ERR_RANGE, "slot %d out of range", slot);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const WsLayout& L = e->lay;
    const size_t first = slot < 0 ? 0 : slot, n = slot < 0 ? c.n_slots : 1;
    CK(cudaMemsetAsync(e->ws + L.rep_counts + first * c.codebook_size * 4, 0, n * c.codebook_size * 4, s));
    CK(cudaMemsetAsync(e->ws + L.rep_hist + first * REP_HIST_MAX * 4, 0, n * REP_HIST_MAX * 4, s));
    CK(cudaMemsetAsync(e->ws + L.rep_head + first * 4, 0, n * 4, s));
    CK(cudaMemsetAsync(e->ws + L.rep_filled + first * 4, 0, n * 4, s));
    return VUIB_OK;
}

extern "C" int32_t vuib_rep_state(VuibEngine* e, int32_t slot, float* counts_out_dev, int32_t* filled_out_dev,
                                  void* stream) {
    if (!e || !counts_out_dev) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    const VuibConfig& c = e->cfg;
    if (slot < 0 || slot >= c.n_slots) return fail(e, VUIB_ERR_RANGE, "slot %d out of range", slot);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CK(cudaMemcpyAsync(counts_out_dev, e->ws + e->lay.rep_counts + (size_t)slot * c.codebook_size * 4,
                       (size_t)c.codebook_size * 4, cudaMemcpyDeviceToDevice, s));
    if (filled_out_dev)
        CK(cudaMemcpyAsync(filled_out_dev, e->ws + e->lay.rep_filled + (size_t)slot * 4, 4, cudaMemcpyDeviceToDevice, s));
    return VUIB_OK;
}

extern "C" int32_t vuib_reset_state(VuibEngine* e, void* stream) {
    if (!e) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    const VuibConfig& c = e->cfg;
    const WsLayout& L = e->lay;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CK(cudaMemsetAsync(e->ws + L.flag, 0, 256, s));
    CK(cudaMemsetAsync(e->ws + L.counters, 0, (size_t)e->R * c.n_kv_heads * 4, s));
    CK(cudaMemsetAsync(e->ws + L.frame_ctr, 0, (size_t)c.n_slots * 4, s));
    CK(cudaMemsetAsync(e->ws + L.tc_counters, 0, 2 * 256 * 4, s));
    return vuib_rep_reset(e, -1, stream);
}

extern "C" int32_t vuib_read_trace(VuibEngine* e, uint64_t* out_host, int32_t n_stamps) {
    if (!e || !out_host) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    if (n_stamps < 1 || n_stamps > TRACE_STAMPS) return fail(e, VUIB_ERR_RANGE, "n_stamps outside [1, %d]", TRACE_STAMPS);
    CK(cudaMemcpy(out_host, e->ws + e->lay.trace, (size_t)n_stamps * 8, cudaMemcpyDeviceToHost));
    return VUIB_OK;
}

extern "C" int32_t vuib_set_wait_limit(VuibEngine* e, uint32_t polls) {
    if (!e) return VUIB_ERR_NULL;
    if (polls < 16) return fail(e, VUIB_ERR_RANGE, "wait limit %u below 16 polls", polls);
    e->spin_limit = polls;
    return VUIB_OK;
}

extern "C" int32_t vuib_debug_withhold_arrival(VuibEngine* e, void* stream) {
    if (!e) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    int32_t minus_one[256];
    for (int i = 0; i < 256; ++i) minus_one[i] = -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CK(cudaMemcpyAsync(e->ws + e->lay.tc_counters, minus_one, sizeof(minus_one), cudaMemcpyHostToDevice, s));
    CK(cudaStreamSynchronize(s));  // the source is a stack array
    return VUIB_OK;
}

extern "C" int32_t vuib_set_seq_len(VuibEngine* e, int32_t slot, int32_t len) {
    if (!e) return VUIB_ERR_NULL;
    if (!e->have_kv) return fail(e, VUIB_ERR_UNBOUND, "bind kv first");
    if (slot < 0 || slot >= e->cfg.n_slots || len < 0 || len > e->cfg.max_seq)
        return fail(e, VUIB_ERR_RANGE, "slot %d / len %d out of range", slot, len);
    CK(cudaMemcpy(e->seq_lens + slot, &len, 4, cudaMemcpyHostToDevice));
    return VUIB_OK;
}

extern "C" int32_t vuib_get_seq_len(VuibEngine* e, int32_t slot, int32_t* len) {
    if (!e || !len) return VUIB_ERR_NULL;
    if (!e->have_kv) return fail(e, VUIB_ERR_UNBOUND, "bind kv first");
    if (slot < 0 || slot >= e->cfg.n_slots) return fail(e, VUIB_ERR_RANGE, "slot %d out of range", slot);
    CK(cudaMemcpy(len, e->seq_lens + slot, 4, cudaMemcpyDeviceToHost));
    return VUIB_OK;
}

extern "C" int32_t vuib_check_device_flag(VuibEngine* e, void* stream) {
    if (!e) return VUIB_ERR_NULL;
    if (!e->have_ws) return fail(e, VUIB_ERR_UNBOUND, "bind the workspace first");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t flag = 0;
    CK(cudaMemcpyAsync(&flag, e->ws + e->lay.flag, 4, cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    if (flag) {
        CK(cudaMemsetAsync(e->ws + e->lay.flag, 0, 4, s));
        // a wait that gave up may have left arrival counters half way: re-arm them with the flag
        CK(cudaMemsetAsync(e->ws + e->lay.tc_counters, 0, 2 * 256 * 4, s));
        CK(cudaMemsetAsync(e->ws + e->lay.counters, 0, (size_t)e->R * e->cfg.n_kv_heads * 4, s));
        return fail(e, VUIB_ERR_DEVICE_FLAG, "device flag 0x%x (1 = slot outside the cache, 2 = position outside [0, max_seq), 4 = code outside the codebook, 16 = a bounded wait inside a kernel ran out)", flag);
    }
    return VUIB_OK;
}

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// A real-time audio thread cannot afford to block on the driver's allocator
// lock, and a plug-in inside a serving process that has already handed all
// device memory to its own pool may be forbidden to call cudaMalloc at all.
// Such callers cannot create the workspace the handle-based API needs, so this
// entry point keeps the split-KV partial results and the per-(row, kv head)
// arrival counters in a fixed array that is part of the loaded module.  Every
// GPU that loads the library holds these ~529 KB until the process exits.
//
// In host code `g_na_scratch` is only a stand-in for the symbol, not a device
// address, so the address the kernel gets comes from cudaGetSymbolAddress, asked
// once per device (with that device current) on the first call there.
// ---------------------------------------------------------------------------
#define VUIB_NA_MAX_ROWS 8
#define VUIB_NA_MAX_HEADS 16
#define VUIB_NA_MAX_SEQ 2048
#define VUIB_NA_MAX_DEVICES 64
constexpr size_t NA_PART_BYTES = (size_t)VUIB_NA_MAX_ROWS * VUIB_NA_MAX_HEADS *
                                 (VUIB_NA_MAX_SEQ / ATT_SPLIT) * PART_STRIDE * sizeof(float);
constexpr size_t NA_COUNTER_BYTES = (size_t)VUIB_NA_MAX_ROWS * VUIB_NA_MAX_HEADS * sizeof(int32_t);
static_assert(NA_PART_BYTES % 256 == 0, "counter block must stay 256-byte aligned");

static __device__ __align__(256) unsigned char g_na_scratch[NA_PART_BYTES + NA_COUNTER_BYTES];

static std::mutex g_na_mutex;
static void* g_na_dev_ptr[VUIB_NA_MAX_DEVICES];  // per device: address of g_na_scratch there

static int32_t na_fail(char* err, size_t n, int32_t code, const char* fmt, ...) {
    if (err && n) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, n, fmt, ap);
        va_end(ap);
    }
    return code;
}

extern "C" int32_t vuib_attention_noalloc(int32_t n_heads, int32_t n_kv_heads, int32_t max_seq,
                                          int32_t n_rows, const void* q_dev, const void* k_cache_dev,
                                          const void* v_cache_dev, const int32_t* row_slot_dev,
                                          const int32_t* row_pos_dev, void* out_dev, void* stream,
                                          char* err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (!q_dev || !k_cache_dev || !v_cache_dev || !row_slot_dev || !row_pos_dev || !out_dev)
        return na_fail(err, err_len, VUIB_ERR_NULL, "a required pointer is NULL");
    if (n_rows < 1 || n_rows > VUIB_NA_MAX_ROWS)
        return na_fail(err, err_len, VUIB_ERR_RANGE, "n_rows %d outside [1, %d]: the built-in scratch holds "
                       "%d rows; use vuib_attention with a workspace for more", n_rows, VUIB_NA_MAX_ROWS,
                       VUIB_NA_MAX_ROWS);
    if (max_seq < 1 || max_seq > VUIB_NA_MAX_SEQ)
        return na_fail(err, err_len, VUIB_ERR_RANGE, "max_seq %d outside [1, %d] (built-in scratch limit)",
                       max_seq, VUIB_NA_MAX_SEQ);
    if (n_heads < 1 || n_heads > VUIB_NA_MAX_HEADS || n_kv_heads < 1 || n_heads % n_kv_heads != 0 ||
        n_heads / n_kv_heads > 2)
        return na_fail(err, err_len, VUIB_ERR_RANGE, "n_heads %d / n_kv_heads %d unsupported (at most %d query "
                       "heads, 1 or 2 per kv head)", n_heads, n_kv_heads, VUIB_NA_MAX_HEADS);
    int dev = -1;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess || dev < 0 || dev >= VUIB_NA_MAX_DEVICES)
        return na_fail(err, err_len, VUIB_ERR_CUDA, "cudaGetDevice: %s (device %d)", cudaGetErrorString(rc), dev);
    void* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_na_mutex);
        if (!g_na_dev_ptr[dev]) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            rc = cudaGetSymbolAddress(&p, g_na_scratch);
            if (rc != cudaSuccess || !p)
                return na_fail(err, err_len, VUIB_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(rc));
            g_na_dev_ptr[dev] = p;
        }
        base = g_na_dev_ptr[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char* b = static_cast<unsigned char*>(base);
    // the array keeps the previous call's contents: the arrival counters must start at zero
    rc = cudaMemsetAsync(b + NA_PART_BYTES, 0, NA_COUNTER_BYTES, s);
    if (rc != cudaSuccess)
        return na_fail(err, err_len, VUIB_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(rc));
    const int S = (max_seq + ATT_SPLIT - 1) / ATT_SPLIT;
    AttnArgs aa{static_cast<const bf16*>(q_dev), static_cast<const bf16*>(k_cache_dev),
                static_cast<const bf16*>(v_cache_dev), row_slot_dev, row_pos_dev,
                reinterpret_cast<float*>(b), reinterpret_cast<int32_t*>(b + NA_PART_BYTES),
                static_cast<bf16*>(out_dev), n_heads, n_kv_heads, max_seq, S, nullptr, 0, nullptr};
    k_attn_decode<<<dim3(S, n_kv_heads, n_rows), ATT_THREADS, 0, s>>>(aa);
    rc = cudaGetLastError();
    if (rc != cudaSuccess)
        return na_fail(err, err_len, VUIB_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(rc));
    return VUIB_OK;
}
