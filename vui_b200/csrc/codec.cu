// Host side of the streaming codec decode: workspace layout, weight binding and the launch
// sequence of one frame (kernels in codec_kernels.cuh).  Entry points: include/vuib200.h,
// section "Streaming codec decode".
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "../../include/vuib200.h"
#include "codec_kernels.cuh"

using namespace vuic;

namespace {

constexpr int HD = 64;
constexpr int UP_T[3] = {1, 2, 4};   // columns per frame before / after each x2 stage

struct ConvState { size_t off; int elems; };   // [2][elems] floats at ws + off

// activated input of a k = 7 convolution: [2 parities][C][ld], P history columns in front (codec_kernels.cuh)
struct PadBuf { size_t off; int ld, P; long long pstride; };

struct Layout {
    size_t ctr, tile_ctr, state_lo, state_hi;   // [0, state_hi) is what a reset zeroes
    ConvState pre_conv, dw[2], dec_in;
    PadBuf res_in[4][3], fin_in;                // inputs of the residual units' first convolutions, of the last conv
    size_t partial[4];                          // transposed-convolution partials [Cout][rate]
    size_t kc, vc;                              // [layers][heads][max_seq][64]
    size_t h0, y1, x, qkv, attn, g, lat, u[2], z, a4, d0, d0a, p, y[4], ya[4], r1, part;
    size_t total;
    int C[5], T[5];                             // channels / columns after decoder.0 and after each block
};

}  // namespace

struct VuibCodec {
    VuibCodecConfig cfg;
    VuibCodecWeights w;
    Layout lay;
    unsigned char* ws;
    bool have_ws, have_w;
    int64_t launches;
    int max_part_floats;
    char err[256];
};

namespace {

int32_t fail(VuibCodec* c, int32_t code, const char* fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof(c->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

bool pdl_enabled() {
    static int v = -1;
    if (v < 0) v = getenv("VUIB_NO_PDL") ? 0 : 1;
    return v == 1;
}

template <class Arg>
cudaError_t launch(VuibCodec* c, void (*kern)(Arg), dim3 grid, dim3 block, size_t smem, cudaStream_t s, const Arg& arg) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
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
    c->launches++;
    return cudaLaunchKernelEx(&cfg, kern, arg);
}

template <class T>
T* wsp(VuibCodec* c, size_t off) { return reinterpret_cast<T*>(c->ws + off); }

size_t take(size_t& cur, size_t bytes) {
    size_t o = cur;
    cur += (bytes + 255) & ~size_t(255);
    return o;
}

// K-split of a tiled convolution: about two CTAs per SM, whole staging steps per split, at most 16 splits
void pick_split(int Cin, int Cout, int T, int cc, int* splits, int* ci_per_split) {
    int tiles = ((T + CT_T - 1) / CT_T) * (Cout / CT_CO);
    int want = (296 + tiles - 1) / tiles;
    int max_s = Cin / cc < 16 ? Cin / cc : 16;   // the last-arriving CTA adds the partial tiles one after the other
    if (want > max_s) want = max_s;
    if (want < 1) want = 1;
    int per = ((Cin + want - 1) / want + cc - 1) / cc * cc;
    *ci_per_split = per;
    *splits = (Cin + per - 1) / per;
}

int part_floats(int Cin, int Cout, int T, int cc) {
    int s, per;
    pick_split(Cin, Cout, T, cc, &s, &per);
    return s > 1 ? s * ((T + CT_T - 1) / CT_T) * (Cout / CT_CO) * CT_CO * CT_T : 0;
}

void make_layout(VuibCodec* c) {
    const VuibCodecConfig& g = c->cfg;
    Layout& L = c->lay;
    size_t cur = 0;
    const int lat = g.latent_dim;
    L.C[0] = g.decoder_dim;
    L.T[0] = UP_T[2];
    for (int b = 0; b < 4; ++b) { L.C[b + 1] = L.C[b] / 2; L.T[b + 1] = L.T[b] * g.rates[b]; }

    L.ctr = take(cur, 16 * sizeof(int));
    L.tile_ctr = take(cur, 4096 * sizeof(int));
    L.state_lo = cur;
    auto st = [&](int elems) { ConvState s{take(cur, 2 * (size_t)elems * 4), elems}; return s; };
    auto padbuf = [&](int C, int T, int P) {
        PadBuf b;
        b.P = P;
        b.ld = (P + T + 3) / 4 * 4 + 4;
        b.pstride = (long long)C * b.ld;
        b.off = take(cur, 2 * (size_t)b.pstride * 4);
        return b;
    };
    L.pre_conv = st(g.vq_dim * 2);
    for (int i = 0; i < 2; ++i) L.dw[i] = st(lat * 6);
    L.dec_in = st(lat * 6);
    const int dil[3] = {1, 3, 9};
    for (int b = 0; b < 4; ++b) {
        L.partial[b] = take(cur, (size_t)L.C[b + 1] * g.rates[b] * 4);
        for (int r = 0; r < 3; ++r) L.res_in[b][r] = padbuf(L.C[b + 1], L.T[b + 1], 6 * dil[r]);
    }
    L.fin_in = padbuf(L.C[4], L.T[4], 6);
    L.state_hi = cur;
    size_t kv = (size_t)g.n_layers * g.n_heads * g.max_seq * HD * 4;
    L.kc = take(cur, kv);
    L.vc = take(cur, kv);
    L.h0 = take(cur, g.vq_dim * 4);
    L.y1 = take(cur, lat * 4);
    L.x = take(cur, g.d_model * 4);
    L.qkv = take(cur, 3 * g.n_heads * HD * 4);
    L.attn = take(cur, g.n_heads * HD * 4);
    L.g = take(cur, g.mlp_dim * 4);
    L.lat = take(cur, lat * 4);
    L.u[0] = take(cur, lat * 2 * 4);
    L.u[1] = take(cur, lat * 4 * 4);
    L.z = take(cur, lat * 4 * 4);
    L.a4 = take(cur, (size_t)lat * 4 * 4 * 4);
    L.d0 = take(cur, (size_t)L.C[0] * L.T[0] * 4);
    L.d0a = take(cur, (size_t)L.C[0] * L.T[0] * 4);
    size_t pmax = 0, ymax = 0;
    int part_max = 1;
    for (int b = 0; b < 4; ++b) {
        const int C = L.C[b + 1], T = L.T[b + 1];
        size_t rows = (size_t)C * 2 * g.rates[b];
        if (rows * L.T[b] > pmax) pmax = rows * L.T[b];
        L.y[b] = take(cur, (size_t)C * T * 4);
        L.ya[b] = take(cur, (size_t)C * T * 4);     // activated copy for the next block's transposed convolution
        if ((size_t)C * T > ymax) ymax = (size_t)C * T;
        int p7 = part_floats(C, C, T, 8), p1 = part_floats(C, C, T, 32);
        int pt = b > 0 ? part_floats(L.C[b], (int)rows, L.T[b], 32) : 0;
        if (p7 > part_max) part_max = p7;
        if (p1 > part_max) part_max = p1;
        if (pt > part_max) part_max = pt;
    }
    L.p = take(cur, pmax * 4);
    L.r1 = take(cur, ymax * 4);
    c->max_part_floats = part_max;
    L.part = take(cur, (size_t)part_max * 4);
    L.total = cur;
}

#define CK(call)                                                                              \
    do {                                                                                      \
        cudaError_t _err = (call);                                                            \
        if (_err != cudaSuccess)                                                              \
            return fail(c, VUIB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(_err));  \
    } while (0)

// ---- launch helpers ---------------------------------------------------------------------------
template <int KW, int T, bool DUAL>
cudaError_t rows_launch(VuibCodec* c, RowsArgs a, cudaStream_t s) {
    // enough warps for every SM: S warps share a row while rows * S is short of ~16 warps per SM
    const int k4 = a.Cin * KW / 4;
    int S = 1;
    while (S < 8 && a.rows * S < 2368 && k4 % (64 * S) == 0) S *= 2;
    a.ksplit = S;
    int rpp = 8 / S, grid = (a.rows + rpp - 1) / rpp;
    if (grid > 592) grid = 592;
    size_t smem = (size_t)a.Cin * (KW == 1 ? T : (KW - 1 + T)) * 4;
    return launch(c, k_crows<KW, T, DUAL>, dim3(grid), dim3(256), smem, s, a);
}

cudaError_t rows(VuibCodec* c, int KW, int T, const RowsArgs& a, cudaStream_t s) {
    const bool dual = a.w2 != nullptr;
    if (KW == 1 && T == 1) return dual ? rows_launch<1, 1, true>(c, a, s) : rows_launch<1, 1, false>(c, a, s);
    if (KW == 1 && T == 2 && !dual) return rows_launch<1, 2, false>(c, a, s);
    if (KW == 1 && T == 4 && !dual) return rows_launch<1, 4, false>(c, a, s);
    if (KW == 3 && T == 1 && !dual) return rows_launch<3, 1, false>(c, a, s);
    if (KW == 7 && T == 4 && !dual) return rows_launch<7, 4, false>(c, a, s);
    return cudaErrorInvalidValue;
}

RowsArgs rows_args(VuibCodec* c, const float* w, const float* bias, const float* x, int x_cs, int x_ts, int Cin,
                   int n_rows, float* y, int y_rs, int y_ts) {
    RowsArgs a = {};
    a.w = w; a.bias = bias; a.x = x; a.x_cs = x_cs; a.x_ts = x_ts; a.Cin = Cin; a.rows = n_rows;
    a.ctr = wsp<int>(c, c->lay.ctr);
    a.pro = PRO_NONE; a.epi = EPI_BIAS; a.eps = c->cfg.norm_eps;
    a.y = y; a.row_div = 1; a.y_rs = y_rs; a.y_js = 0; a.y_ts = y_ts;
    return a;
}

struct TileIn { const float* xa; long long pstride; int ld, P; };

TileIn plain_in(const float* x, int T) { return TileIn{x, 0, T, 0}; }
TileIn pad_in(VuibCodec* c, const PadBuf& b) { return TileIn{wsp<float>(c, b.off), b.pstride, b.ld, b.P}; }

ActOut act_into_pad(VuibCodec* c, const PadBuf& b, const VuibSnakeW& a) {
    return ActOut{wsp<float>(c, b.off), b.pstride, b.ld, b.P, a.ea, a.ib};
}
ActOut act_into_plain(float* dst, int T, const VuibSnakeW& a) { return ActOut{dst, 0, T, 0, a.ea, a.ib}; }

cudaError_t tile(VuibCodec* c, int KW, const float* wt, const float* bias, TileIn in, const float* res, float* y,
                 ActOut act, int Cin, int Cout, int T, int dil, cudaStream_t s) {
    const int cc = KW == 1 ? 32 : 8;
    if (Cout % CT_CO || Cin % cc || T % 4 || in.ld % 4) return cudaErrorInvalidValue;
    TileArgs a = {};
    a.wt = wt; a.bias = bias; a.xa = in.xa; a.x_pstride = in.pstride; a.x_ld = in.ld; a.P = in.P;
    a.res = res; a.y = y; a.act = act;
    a.part = wsp<float>(c, c->lay.part); a.tile_ctr = wsp<int>(c, c->lay.tile_ctr);
    a.ctr = wsp<int>(c, c->lay.ctr);
    a.Cin = Cin; a.Cout = Cout; a.T = T; a.dil = dil;
    pick_split(Cin, Cout, T, cc, &a.splits, &a.ci_per_split);
    dim3 grid((T + CT_T - 1) / CT_T, Cout / CT_CO, a.splits);
    if ((int)(grid.x * grid.y) > 4096 ||
        (a.splits > 1 && (int)(a.splits * grid.x * grid.y * CT_CO * CT_T) > c->max_part_floats) ||
        in.P != (KW - 1) * dil)
        return cudaErrorInvalidValue;
    if (KW == 7) return launch(c, k_ctile<7>, grid, dim3(CT_THREADS), ct_smem_bytes<7>(), s, a);
    if (KW == 1) return launch(c, k_ctile<1>, grid, dim3(CT_THREADS), ct_smem_bytes<1>(), s, a);
    return cudaErrorInvalidValue;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
extern "C" int32_t vuib_codec_create(const VuibCodecConfig* cfg, VuibCodec** out) {
    if (!cfg || !out) return VUIB_ERR_NULL;
    *out = nullptr;
    const VuibCodecConfig& g = *cfg;
    bool ok = g.n_q == 16 && g.codebook_size == 2048 && g.codebook_dim == 256 && g.vq_dim == 512 &&
              g.latent_dim == 1024 && g.d_model == 512 && g.n_heads == 16 && g.mlp_dim == 1024 &&
              g.n_layers >= 1 && g.n_layers <= VUIB_CODEC_LAYERS && g.decoder_dim == 1536 &&
              g.rates[0] == 8 && g.rates[1] == 5 && g.rates[2] == 4 && g.rates[3] == 3;
    if (!ok) return VUIB_ERR_SHAPE;
    if (g.max_seq < 1 || g.max_seq > 256) return VUIB_ERR_RANGE;
    VuibCodec* c = new (std::nothrow) VuibCodec();
    if (!c) return VUIB_ERR_NULL;
    memset(c, 0, sizeof(*c));
    c->cfg = g;
    make_layout(c);
    *out = c;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_destroy(VuibCodec* c) {
    delete c;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_last_error(VuibCodec* c, char* buf, size_t n) {
    if (!c || !buf || n == 0) return VUIB_ERR_NULL;
    strncpy(buf, c->err, n - 1);
    buf[n - 1] = 0;
    return VUIB_OK;
}

extern "C" int64_t vuib_codec_launch_count(VuibCodec* c) { return c ? c->launches : 0; }

extern "C" int32_t vuib_codec_workspace_bytes(VuibCodec* c, size_t* bytes) {
    if (!c || !bytes) return VUIB_ERR_NULL;
    *bytes = c->lay.total;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_bind_workspace(VuibCodec* c, void* dev, size_t bytes) {
    if (!c || !dev) return VUIB_ERR_NULL;
    if (bytes < c->lay.total || ((uintptr_t)dev & 255))
        return fail(c, VUIB_ERR_WORKSPACE, "codec workspace needs %zu bytes, 256-byte aligned; got %zu at %p",
                    c->lay.total, bytes, dev);
    c->ws = static_cast<unsigned char*>(dev);
    c->have_ws = true;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_bind_weights(VuibCodec* c, const VuibCodecWeights* w) {
    if (!c || !w) return VUIB_ERR_NULL;
    // every pointer of the struct must be set (the struct is pointers only), except layers beyond n_layers
    VuibCodecWeights tmp = *w;
    for (int l = c->cfg.n_layers; l < VUIB_CODEC_LAYERS; ++l) tmp.layer[l] = tmp.layer[0];
    const void* const* p = reinterpret_cast<const void* const*>(&tmp);
    for (size_t i = 0; i < sizeof(tmp) / sizeof(void*); ++i)
        if (!p[i]) return fail(c, VUIB_ERR_NULL, "codec weight pointer #%zu is NULL", i);
    for (size_t i = 0; i < sizeof(tmp) / sizeof(void*); ++i)
        if ((uintptr_t)p[i] & 15) return fail(c, VUIB_ERR_WORKSPACE, "codec weight pointer #%zu is not 16-byte aligned", i);
    c->w = *w;
    c->have_w = true;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_reset(VuibCodec* c, void* stream) {
    if (!c) return VUIB_ERR_NULL;
    if (!c->have_ws) return fail(c, VUIB_ERR_UNBOUND, "codec workspace not bound");
    // counters, tile counters and every streaming state are contiguous from the start of the block;
    // the transformer KV needs no clearing: positions beyond the counter are never read
    CK(cudaMemsetAsync(c->ws, 0, c->lay.state_hi, static_cast<cudaStream_t>(stream)));
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_position(VuibCodec* c, int32_t* pos, void* stream) {
    if (!c || !pos) return VUIB_ERR_NULL;
    if (!c->have_ws) return fail(c, VUIB_ERR_UNBOUND, "codec workspace not bound");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CK(cudaMemcpyAsync(pos, wsp<int>(c, c->lay.ctr) + CTR_POS, sizeof(int), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_check_flag(VuibCodec* c, void* stream) {
    if (!c) return VUIB_ERR_NULL;
    if (!c->have_ws) return fail(c, VUIB_ERR_UNBOUND, "codec workspace not bound");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int flag = 0;
    CK(cudaMemcpyAsync(&flag, wsp<int>(c, c->lay.ctr) + CTR_FLAG, sizeof(int), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    if (!flag) return VUIB_OK;
    CK(cudaMemsetAsync(wsp<int>(c, c->lay.ctr) + CTR_FLAG, 0, sizeof(int), s));
    CK(cudaStreamSynchronize(s));
    return fail(c, VUIB_ERR_DEVICE_FLAG, "codec device flag 0x%x:%s%s", flag,
                (flag & FLAG_BAD_CODE) ? " code outside [0, 2048)" : "",
                (flag & FLAG_POS_OVERFLOW) ? " transformer position beyond max_seq" : "");
}

extern "C" int32_t vuib_codec_read_tap(VuibCodec* c, int32_t which, float* out_host, int32_t n, void* stream) {
    if (!c || !out_host) return VUIB_ERR_NULL;
    if (!c->have_ws) return fail(c, VUIB_ERR_UNBOUND, "codec workspace not bound");
    const Layout& L = c->lay;
    size_t off;
    int have;
    switch (which) {
        case 0: off = L.h0; have = c->cfg.vq_dim; break;
        case 1: off = L.lat; have = c->cfg.latent_dim; break;
        case 2: off = L.u[1]; have = c->cfg.latent_dim * 4; break;
        case 3: off = L.d0; have = L.C[0] * L.T[0]; break;
        case 4: case 5: case 6: case 7: off = L.y[which - 4]; have = L.C[which - 3] * L.T[which - 3]; break;
        default: return fail(c, VUIB_ERR_RANGE, "tap %d does not exist", which);
    }
    if (n < 1 || n > have) return fail(c, VUIB_ERR_RANGE, "tap %d holds %d floats, asked for %d", which, have, n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CK(cudaMemcpyAsync(out_host, c->ws + off, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_decode_frame(VuibCodec* c, const int64_t* codes_dev, int32_t n_q, float* audio_out_dev,
                                           void* stream) {
    if (!c || !codes_dev || !audio_out_dev) return VUIB_ERR_NULL;
    if (!c->have_ws || !c->have_w) return fail(c, VUIB_ERR_UNBOUND, "codec workspace or weights not bound");
    if (n_q < 1 || n_q > c->cfg.n_q) return fail(c, VUIB_ERR_RANGE, "n_q = %d outside [1, %d]", n_q, c->cfg.n_q);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const VuibCodecConfig& g = c->cfg;
    const VuibCodecWeights& w = c->w;
    const Layout& L = c->lay;
    int* ctr = wsp<int>(c, L.ctr);
    const int lat = g.latent_dim, D = g.d_model, HH = g.n_heads * HD;

    {   // quantizer.decode
        EmbedArgs a = {};
        a.codes = reinterpret_cast<const long long*>(codes_dev);
        a.n_q = n_q;
        for (int q = 0; q < 16; ++q) a.table[q] = w.codebook[q];
        a.sem_proj = w.sem_proj; a.acq_proj = w.acq_proj; a.out = wsp<float>(c, L.h0); a.ctr = ctr;
        CK(launch(c, k_cq_embed, dim3(g.vq_dim / 8), dim3(256), 0, s, a));
    }
    {   // pre_conv (k = 3)
        RowsArgs a = rows_args(c, w.pre_conv.w, w.pre_conv.b, wsp<float>(c, L.h0), 1, 0, g.vq_dim, lat,
                               wsp<float>(c, L.y1), 1, 0);
        a.state = wsp<float>(c, L.pre_conv.off);
        CK(rows(c, 3, 1, a, s));
    }
    {   // pre_transformer.input_proj
        RowsArgs a = rows_args(c, w.in_proj.w, w.in_proj.b, wsp<float>(c, L.y1), 1, 0, lat, D, wsp<float>(c, L.x), 1, 0);
        CK(rows(c, 1, 1, a, s));
    }
    for (int l = 0; l < g.n_layers; ++l) {
        const VuibCodecLayerW& lw = w.layer[l];
        {
            RowsArgs a = rows_args(c, lw.wqkv, nullptr, wsp<float>(c, L.x), 1, 0, D, 3 * HH, wsp<float>(c, L.qkv), 1, 0);
            a.pro = PRO_RMSNORM; a.p0 = lw.ln1;
            CK(rows(c, 1, 1, a, s));
        }
        {
            CAttnArgs a = {};
            a.qkv = wsp<float>(c, L.qkv);
            a.kc = wsp<float>(c, L.kc) + (size_t)l * g.n_heads * g.max_seq * HD;
            a.vc = wsp<float>(c, L.vc) + (size_t)l * g.n_heads * g.max_seq * HD;
            a.cos_t = w.rope_cos; a.sin_t = w.rope_sin; a.out = wsp<float>(c, L.attn); a.ctr = ctr;
            a.H = g.n_heads; a.max_seq = g.max_seq;
            CK(launch(c, k_ct_attn, dim3(g.n_heads), dim3(128), 0, s, a));
        }
        {
            RowsArgs a = rows_args(c, lw.wo, nullptr, wsp<float>(c, L.attn), 1, 0, HH, D, wsp<float>(c, L.x), 1, 0);
            a.epi = EPI_SCALE_RES; a.scale = lw.attn_scale; a.res = wsp<float>(c, L.x);
            CK(rows(c, 1, 1, a, s));
        }
        {
            RowsArgs a = rows_args(c, lw.gate, nullptr, wsp<float>(c, L.x), 1, 0, D, g.mlp_dim, wsp<float>(c, L.g), 1, 0);
            a.w2 = lw.up; a.pro = PRO_RMSNORM; a.p0 = lw.ln2; a.epi = EPI_SILU_MUL;
            CK(rows(c, 1, 1, a, s));
        }
        {
            RowsArgs a = rows_args(c, lw.down, nullptr, wsp<float>(c, L.g), 1, 0, g.mlp_dim, D, wsp<float>(c, L.x), 1, 0);
            a.epi = EPI_SCALE_RES; a.scale = lw.mlp_scale; a.res = wsp<float>(c, L.x);
            CK(rows(c, 1, 1, a, s));
        }
    }
    {   // pre_transformer.norm + output_proj
        RowsArgs a = rows_args(c, w.out_proj.w, w.out_proj.b, wsp<float>(c, L.x), 1, 0, D, lat, wsp<float>(c, L.lat), 1, 0);
        a.pro = PRO_RMSNORM; a.p0 = w.norm;
        CK(rows(c, 1, 1, a, s));
    }
    const float* cur = wsp<float>(c, L.lat);   // [1024][Tin] channel-major
    for (int i = 0; i < 2; ++i) {
        const VuibUpStageW& uw = w.stage[i];
        const int Tin = UP_T[i], Tout = UP_T[i + 1];
        float* u = wsp<float>(c, L.u[i]);
        {   // transposed convolution, kernel = stride = 2: rows (co, j) scatter to column 2 t + j
            RowsArgs a = rows_args(c, uw.up.w, uw.up.b, cur, Tin, 1, lat, lat * 2, u, Tout, 2);
            a.row_div = 2; a.y_js = 1;
            CK(rows(c, 1, Tin, a, s));
        }
        {
            DwLnArgs a = {};
            a.x = u; a.w = uw.dw.w; a.b = uw.dw.b; a.ln_w = uw.ln_w; a.ln_b = uw.ln_b;
            a.state = wsp<float>(c, L.dw[i].off); a.ctr = ctr; a.z = wsp<float>(c, L.z); a.C = lat; a.T = Tout;
            CK(launch(c, k_dwconv_ln, dim3(Tout), dim3(256), 0, s, a));
        }
        {   // pwconv1 + GELU, time-major in and out
            RowsArgs a = rows_args(c, uw.pw1.w, uw.pw1.b, wsp<float>(c, L.z), 1, lat, lat, lat * 4,
                                   wsp<float>(c, L.a4), 1, lat * 4);
            a.epi = EPI_GELU;
            CK(rows(c, 1, Tout, a, s));
        }
        {   // residual + gamma * pwconv2, back to channel-major, in place on u
            RowsArgs a = rows_args(c, uw.pw2.w, uw.pw2.b, wsp<float>(c, L.a4), 1, lat * 4, lat * 4, lat, u, Tout, 1);
            a.epi = EPI_SCALE_RES; a.scale = uw.gamma; a.res = u;
            CK(rows(c, 1, Tout, a, s));
        }
        cur = u;
    }
    {   // decoder.0 (k = 7) on 4 columns
        RowsArgs a = rows_args(c, w.dec_in.w, w.dec_in.b, cur, 4, 1, lat, L.C[0], wsp<float>(c, L.d0), 4, 1);
        a.state = wsp<float>(c, L.dec_in.off);
        a.y_act = wsp<float>(c, L.d0a); a.act_ea = w.block[0].act.ea; a.act_ib = w.block[0].act.ib;
        CK(rows(c, 7, 4, a, s));
    }
    cur = wsp<float>(c, L.d0a);  // decoder.0's output with the first block's SnakeBeta already applied
    const int dil[3] = {1, 3, 9};
    const ActOut no_act = {};
    for (int b = 0; b < 4; ++b) {
        const VuibDecBlockW& bw = w.block[b];
        const int Cin = L.C[b], Cout = L.C[b + 1], Tin = L.T[b], Tout = L.T[b + 1], rate = g.rates[b];
        const int prow = Cout * 2 * rate;
        float* p = wsp<float>(c, L.p);
        float* y = wsp<float>(c, L.y[b]);
        float* r1 = wsp<float>(c, L.r1);
        if (b == 0) {
            RowsArgs a = rows_args(c, bw.up.w, nullptr, cur, Tin, 1, Cin, prow, p, Tin, 1);
            CK(rows(c, 1, Tin, a, s));
        } else {   // the previous block left its output activated in ya[b - 1]
            CK(tile(c, 1, bw.up.w, nullptr, plain_in(wsp<float>(c, L.ya[b - 1]), Tin), nullptr, p, no_act, Cin, prow, Tin,
                    1, s));
        }
        {
            OlaArgs a = {};
            a.p = p; a.bias = bw.up.b; a.partial = wsp<float>(c, L.partial[b]); a.y = y;
            a.act = act_into_pad(c, L.res_in[b][0], bw.res[0].act1); a.ctr = ctr;
            a.Cout = Cout; a.s = rate; a.Tin = Tin;
            CK(launch(c, k_overlap_add, dim3((Cout * Tout + 255) / 256), dim3(256), 0, s, a));
        }
        for (int r = 0; r < 3; ++r) {
            const VuibResUnitW& rw = bw.res[r];
            // conv1: activated padded input -> r1 = act2(conv1(...)), only the activated form is needed
            CK(tile(c, 7, rw.conv1.w, rw.conv1.b, pad_in(c, L.res_in[b][r]), nullptr, nullptr,
                    act_into_plain(r1, Tout, rw.act2), Cout, Cout, Tout, dil[r], s));
            // conv2: y += conv2(r1); the activated copy goes to whoever consumes y next
            ActOut nxt = r < 2   ? act_into_pad(c, L.res_in[b][r + 1], bw.res[r + 1].act1)
                         : b < 3 ? act_into_plain(wsp<float>(c, L.ya[b]), Tout, w.block[b + 1].act)
                                 : act_into_pad(c, L.fin_in, w.final_act);
            CK(tile(c, 1, rw.conv2.w, rw.conv2.b, plain_in(r1, Tout), y, y, nxt, Cout, Cout, Tout, 1, s));
        }
    }
    {
        FinalArgs a = {};
        a.xa = wsp<float>(c, L.fin_in.off); a.x_pstride = L.fin_in.pstride; a.x_ld = L.fin_in.ld;
        a.w = w.final_conv.w; a.bias = w.final_conv.b; a.ctr = ctr; a.audio = audio_out_dev; a.C = L.C[4]; a.T = L.T[4];
        CK(launch(c, k_final_conv, dim3((a.T + 31) / 32), dim3(128), (size_t)a.C * 40 * 4, s, a));
    }
    CK(launch(c, k_advance, dim3(1), dim3(32), 0, s, ctr));
    return VUIB_OK;
}
