// Host side of the codec encoder: workspace layout, weight binding and the launch sequence of one encode call
// (kernels in codec_enc_kernels.cuh).  Entry points: include/vuib200.h, section "Codec encoder".
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "../../include/vuib200.h"
#include "codec_enc_kernels.cuh"

using namespace vuie;

struct VuibCodecEnc {
    VuibCodecEncConfig cfg;
    VuibCodecEncWeights w;
    unsigned char* ws;
    bool have_ws, have_w;
    int64_t launches;
    size_t off_a, off_b, off_x, off_n, off_q, off_o, off_g, off_d, off_hs, off_ha, total;
    int last_frames;
    char err[256];
};

namespace {

int32_t fail(VuibCodecEnc* c, int32_t code, const char* fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof(c->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

#define CK(call)                                                                              \
    do {                                                                                      \
        cudaError_t _err = (call);                                                            \
        if (_err != cudaSuccess)                                                              \
            return fail(c, VUIB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(_err));  \
    } while (0)

float* wsf(VuibCodecEnc* c, size_t off) { return reinterpret_cast<float*>(c->ws + off); }

cudaError_t conv(VuibCodecEnc* c, const float* w, const float* bias, const float* x, float* y, int Cin, int Cout, int K,
                 int stride, int Tin, bool elu_in, int epi, const float* res, const float* scale, cudaStream_t s) {
    EConvArgs a = {};
    a.w = w; a.bias = bias; a.x = x; a.res = res; a.scale = scale; a.y = y;
    a.Cin = Cin; a.Cout = Cout; a.K = K; a.stride = stride; a.Tin = Tin; a.Tout = Tin / stride;
    a.elu_in = elu_in ? 1 : 0; a.epi = epi;
    a.cc = K == 1 ? 32 : 8;
    const int XW = EC_T * stride + (K - stride);
    const size_t smem = (size_t)(a.cc * XW + EC_CO * (a.cc * K + 1)) * 4;
    dim3 grid((a.Tout + EC_T - 1) / EC_T, (Cout + EC_CO - 1) / EC_CO);
    c->launches++;
    k_econv<<<grid, EC_THREADS, smem, s>>>(a);
    return cudaGetLastError();
}

}  // namespace

extern "C" int32_t vuib_codec_enc_create(const VuibCodecEncConfig* cfg, VuibCodecEnc** out) {
    if (!cfg || !out) return VUIB_ERR_NULL;
    *out = nullptr;
    const VuibCodecEncConfig& g = *cfg;
    bool ok = g.base_dim == 64 && g.ratios[0] == 4 && g.ratios[1] == 5 && g.ratios[2] == 6 && g.ratios[3] == 8 &&
              g.d_model == 512 && g.n_heads == 8 && g.mlp_dim == 2048 && g.n_layers >= 1 &&
              g.n_layers <= VUIB_CODEC_LAYERS;
    if (!ok) return VUIB_ERR_SHAPE;
    if (g.max_samples < 1920 || g.max_samples % 1920 || g.max_samples > 480000) return VUIB_ERR_RANGE;
    VuibCodecEnc* c = new (std::nothrow) VuibCodecEnc();
    if (!c) return VUIB_ERR_NULL;
    memset(c, 0, sizeof(*c));
    c->cfg = g;
    size_t cur = 0;
    auto take = [&](size_t floats) { size_t o = cur; cur += (floats * 4 + 255) & ~size_t(255); return o; };
    const size_t T0 = g.max_samples, T25 = T0 / 960, T12 = T0 / 1920;
    c->off_a = take(64 * T0);        // stage outputs alternate between a and b (largest: 64 x T0)
    c->off_b = take(64 * T0);
    c->off_x = take(512 * T25);
    c->off_n = take(512 * T25);
    c->off_q = take(3 * 512 * T25);
    c->off_o = take(512 * T25);
    c->off_g = take((size_t)g.mlp_dim * T25);
    c->off_d = take(512 * T12);
    c->off_hs = take(256 * T12);
    c->off_ha = take(256 * T12);
    c->total = cur;
    *out = c;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_enc_destroy(VuibCodecEnc* c) {
    delete c;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_enc_last_error(VuibCodecEnc* c, char* buf, size_t n) {
    if (!c || !buf || n == 0) return VUIB_ERR_NULL;
    strncpy(buf, c->err, n - 1);
    buf[n - 1] = 0;
    return VUIB_OK;
}

extern "C" int64_t vuib_codec_enc_launch_count(VuibCodecEnc* c) { return c ? c->launches : 0; }

extern "C" int32_t vuib_codec_enc_workspace_bytes(VuibCodecEnc* c, size_t* bytes) {
    if (!c || !bytes) return VUIB_ERR_NULL;
    *bytes = c->total;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_enc_bind_workspace(VuibCodecEnc* c, void* dev, size_t bytes) {
    if (!c || !dev) return VUIB_ERR_NULL;
    if (bytes < c->total || ((uintptr_t)dev & 255))
        return fail(c, VUIB_ERR_WORKSPACE, "encoder workspace needs %zu bytes, 256-byte aligned; got %zu at %p", c->total,
                    bytes, dev);
    c->ws = static_cast<unsigned char*>(dev);
    c->have_ws = true;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_enc_bind_weights(VuibCodecEnc* c, const VuibCodecEncWeights* w) {
    if (!c || !w) return VUIB_ERR_NULL;
    VuibCodecEncWeights tmp = *w;
    for (int l = c->cfg.n_layers; l < VUIB_CODEC_LAYERS; ++l) tmp.layer[l] = tmp.layer[0];
    const void* const* p = reinterpret_cast<const void* const*>(&tmp);
    for (size_t i = 0; i < sizeof(tmp) / sizeof(void*); ++i)
        if (!p[i]) return fail(c, VUIB_ERR_NULL, "encoder weight pointer #%zu is NULL", i);
    c->w = *w;
    c->have_w = true;
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_enc_read_latent(VuibCodecEnc* c, float* out_host, int32_t n, void* stream) {
    if (!c || !out_host) return VUIB_ERR_NULL;
    if (!c->have_ws) return fail(c, VUIB_ERR_UNBOUND, "encoder workspace not bound");
    if (n < 1 || n > 512 * c->last_frames) return fail(c, VUIB_ERR_RANGE, "latent holds %d floats", 512 * c->last_frames);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CK(cudaMemcpyAsync(out_host, c->ws + c->off_d, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    return VUIB_OK;
}

extern "C" int32_t vuib_codec_enc_encode(VuibCodecEnc* c, const float* audio_dev, int32_t n_samples, int32_t n_q,
                                         int64_t* codes_out_dev, void* stream) {
    if (!c || !audio_dev || !codes_out_dev) return VUIB_ERR_NULL;
    if (!c->have_ws || !c->have_w) return fail(c, VUIB_ERR_UNBOUND, "encoder workspace or weights not bound");
    if (n_samples < 1920 || n_samples % 1920 || n_samples > c->cfg.max_samples)
        return fail(c, VUIB_ERR_RANGE, "n_samples = %d: need a multiple of 1920 up to %d", n_samples, c->cfg.max_samples);
    if (n_q < 1 || n_q > 16) return fail(c, VUIB_ERR_RANGE, "n_q = %d outside [1, 16]", n_q);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const VuibCodecEncConfig& g = c->cfg;
    const VuibCodecEncWeights& w = c->w;
    float* a = wsf(c, c->off_a);
    float* b = wsf(c, c->off_b);
    int T = n_samples, C = g.base_dim;
    // ---- ConvEncoder (qwen_codec.py:293-311)
    CK(conv(c, w.conv_in.w, w.conv_in.b, audio_dev, a, 1, C, 7, 1, T, false, EE_BIAS, nullptr, nullptr, s));
    for (int i = 0; i < 4; ++i) {
        const int r = g.ratios[i];
        // ResBlock: a += conv1(ELU(conv3(ELU(a))))
        CK(conv(c, w.res[i].c3.w, w.res[i].c3.b, a, b, C, C / 2, 3, 1, T, true, EE_BIAS, nullptr, nullptr, s));
        CK(conv(c, w.res[i].c1.w, w.res[i].c1.b, b, a, C / 2, C, 1, 1, T, true, EE_RES, a, nullptr, s));
        // ELU, strided convolution
        CK(conv(c, w.down[i].w, w.down[i].b, a, b, C, 2 * C, 2 * r, r, T, true, EE_BIAS, nullptr, nullptr, s));
        float* t = a; a = b; b = t;
        C *= 2;
        T /= r;
    }
    float* x = wsf(c, c->off_x);
    CK(conv(c, w.conv_out.w, w.conv_out.b, a, x, C, g.d_model, 3, 1, T, true, EE_BIAS, nullptr, nullptr, s));
    // ---- EncTransformer (314-365) on [512][T], T = 25 Hz frames
    const int D = g.d_model, H = g.n_heads;
    float* nrm = wsf(c, c->off_n);
    float* q = wsf(c, c->off_q);   // [3 * 512][T]: q, k, v
    float* o = wsf(c, c->off_o);
    float* gact = wsf(c, c->off_g);
    for (int l = 0; l < g.n_layers; ++l) {
        const VuibEncLayerW& lw = w.layer[l];
        k_elayernorm<<<(T + 31) / 32, 256, 0, s>>>(x, lw.ln1_w, lw.ln1_b, nrm, D, T);
        c->launches++;
        // q | k | v rows stacked in one matrix: one launch with three times the CTAs
        CK(conv(c, lw.wqkv, nullptr, nrm, q, D, 3 * D, 1, 1, T, false, EE_BIAS, nullptr, nullptr, s));
        k_eattn<<<(H * T + 3) / 4, 128, 0, s>>>(q, q + (size_t)D * T, q + (size_t)2 * D * T, w.rope_cos, w.rope_sin, o, H, T);
        c->launches++;
        CK(conv(c, lw.wo, nullptr, o, x, D, D, 1, 1, T, false, EE_SCALE_RES, x, lw.attn_scale, s));
        k_elayernorm<<<(T + 31) / 32, 256, 0, s>>>(x, lw.ln2_w, lw.ln2_b, nrm, D, T);
        c->launches++;
        CK(conv(c, lw.fc1, nullptr, nrm, gact, D, g.mlp_dim, 1, 1, T, false, EE_GELU, nullptr, nullptr, s));
        CK(conv(c, lw.fc2, nullptr, gact, x, g.mlp_dim, D, 1, 1, T, false, EE_SCALE_RES, x, lw.mlp_scale, s));
    }
    // ---- downsample to 12.5 Hz, project, quantise
    float* d = wsf(c, c->off_d);
    CK(conv(c, w.downsample, nullptr, x, d, D, D, 4, 2, T, false, EE_BIAS, nullptr, nullptr, s));
    T /= 2;
    c->last_frames = T;
    float* hs = wsf(c, c->off_hs);
    float* ha = wsf(c, c->off_ha);
    CK(conv(c, w.sem_in, nullptr, d, hs, D, 256, 1, 1, T, false, EE_BIAS, nullptr, nullptr, s));
    ERvqArgs r = {};
    r.h = hs; r.codes = reinterpret_cast<long long*>(codes_out_dev); r.T = T;
    r.n = 1; r.q0 = 0; r.table[0] = w.codebook[0]; r.norm2[0] = w.codebook_norm2[0];
    k_ervq<<<T, 256, 0, s>>>(r);
    c->launches++;
    if (n_q > 1) {
        CK(conv(c, w.acq_in, nullptr, d, ha, D, 256, 1, 1, T, false, EE_BIAS, nullptr, nullptr, s));
        r.h = ha; r.n = n_q - 1; r.q0 = 1;
        for (int i = 0; i < n_q - 1; ++i) { r.table[i] = w.codebook[1 + i]; r.norm2[i] = w.codebook_norm2[1 + i]; }
        k_ervq<<<T, 256, 0, s>>>(r);
        c->launches++;
    }
    CK(cudaGetLastError());
    return VUIB_OK;
}
