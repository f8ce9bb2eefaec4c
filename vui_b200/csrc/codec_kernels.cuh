// Streaming decode of one codec frame (16 codes -> 1920 samples at 24 kHz) in fp32.
//
// Replaces the single-frame streaming forward of the reference's QwenCodecDecoder
// (src/vui/qwen_codec.py:1191-1224): split residual VQ lookup (200-275), causal
// pre-convolution (45-102), an 8-layer transformer with a fixed 250-position KV
// (882-1076), two x2 upsampling stages (transposed convolution + ConvNeXt block,
// 112-158, 832-848), the BigVGAN-style decoder (851-879: SnakeBeta, overlapping
// transposed convolutions with rates 8,5,4,3, dilated residual units) and the final
// convolution + clamp.  Every causal layer keeps its streaming state (the last
// `pad` input columns of a convolution, the trailing partial of a transposed
// convolution, the transformer's KV and position) in device memory between frames.
//
// Shapes per frame are tiny in time (1, 2, 4 columns) up to the first decoder block
// and long (32 ... 1920 columns) after it, hence two matrix kernels:
//   k_crows : a warp per output row streams that row's weights once (HBM bound;
//             all columns of the frame share the pass); prologues RMSNorm / SnakeBeta,
//             epilogues bias / GELU / layer-scale + residual / SiLU-gate / scatter.
//   k_ctile : register-tiled (co x t) convolution with dilation for the long stages,
//             K split over CTAs with an ordered last-arriver reduction.
// Streaming state is double-buffered by frame parity (read [parity], write
// [parity ^ 1]) so no CTA can overwrite history another CTA still reads.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vuic {

constexpr int CTR_FRAME = 0;   // frames decoded since the last reset (its low bit is the state parity)
constexpr int CTR_POS = 1;     // next transformer position
constexpr int CTR_FLAG = 2;    // sticky error bits
constexpr int FLAG_BAD_CODE = 1;
constexpr int FLAG_POS_OVERFLOW = 2;

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// SnakeBeta with precomputed ea = exp(alpha), ib = 1 / (exp(beta) + 1e-9)  (qwen_codec.py:826-829)
__device__ __forceinline__ float snake(float x, float ea, float ib) {
    float s = sinf(x * ea);
    return x + ib * (s * s);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// block-wide sum for up to 1024 threads; `red` holds 32 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = (l < nw) ? red[l] : 0.f;
    t = warp_sum(t);
    return t;
}

// ---------------------------------------------------------------- quantizer lookup
struct EmbedArgs {
    const long long* codes;      // [n_q]
    int n_q;
    const float* table[16];      // codebook q: (2048, 256); q = 0 semantic, 1.. acoustic
    const float* sem_proj;       // (512, 256)
    const float* acq_proj;       // (512, 256)
    float* out;                  // [512]
    int* ctr;
};

// SplitResidualVQ.decode (qwen_codec.py:231-238, 263-271): sum the code vectors of the semantic and
// of the acoustic codebooks in codebook order, project each sum to 512 channels, add.
__global__ void __launch_bounds__(256) k_cq_embed(EmbedArgs a) {
    __shared__ float s_sem[256], s_acq[256];
    pdl_wait();
    pdl_launch();
    int c = threadIdx.x;
    float sem = 0.f, acq = 0.f;
    for (int q = 0; q < a.n_q; ++q) {
        long long code = a.codes[q];
        if (code < 0 || code >= 2048) {
            if (c == 0) atomicOr(a.ctr + CTR_FLAG, FLAG_BAD_CODE);
            code = code < 0 ? 0 : 2047;
        }
        float v = a.table[q][code * 256 + c];
        if (q == 0) sem += v; else acq += v;
    }
    s_sem[c] = sem;
    s_acq[c] = acq;
    __syncthreads();
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    int row = blockIdx.x * 8 + w;
    float d0 = 0.f, d1 = 0.f;
    for (int k = l; k < 256; k += 32) {
        d0 += a.sem_proj[row * 256 + k] * s_sem[k];
        if (a.n_q > 1) d1 += a.acq_proj[row * 256 + k] * s_acq[k];
    }
    d0 = warp_sum(d0);
    d1 = warp_sum(d1);
    if (l == 0) a.out[row] = d0 + d1;
}

// ---------------------------------------------------------------- warp-per-row matrix kernel
enum { PRO_NONE = 0, PRO_RMSNORM = 1, PRO_SNAKE = 2 };
enum { EPI_BIAS = 0, EPI_GELU = 1, EPI_SCALE_RES = 2, EPI_SILU_MUL = 3 };

struct RowsArgs {
    const float* w;       // [rows][Cin * KW]
    const float* w2;      // second matrix of a gated pair (DUAL) or null
    const float* bias;    // bias[row / row_div] or null
    const float* x;       // input element (ci, t) at x[ci * x_cs + t * x_ts]
    int x_cs, x_ts;
    float* state;         // [2][Cin * (KW-1)] history of the input, or null when KW == 1
    const int* ctr;
    int Cin, rows;
    int pro;              // PRO_*
    const float* p0;      // RMSNorm weight | snake ea
    const float* p1;      // snake ib
    float eps;
    int epi;              // EPI_*
    float* y;             // output (row, t) at y[(row / row_div) * y_rs + (row % row_div) * y_js + t * y_ts]
    int row_div, y_rs, y_js, y_ts;
    const float* scale;   // EPI_SCALE_RES: per-(row / row_div) factor
    const float* res;     // EPI_SCALE_RES: residual, indexed like y
};

// out[row][t] = sum_{ci, j} w[row][ci][j] * X[ci][t + j]  with X = [history | new columns] (causal, dilation 1)
template <int KW, int T, bool DUAL>
__global__ void __launch_bounds__(256) k_crows(RowsArgs a) {
    extern __shared__ float xs[];   // KW == 1: [T][Cin];  KW > 1: [Cin][P], P = KW - 1 + T
    __shared__ float red[32];
    constexpr int PAD = KW - 1, P = PAD + T;
    pdl_wait();
    pdl_launch();
    const int tid = threadIdx.x, Cin = a.Cin;
    const int parity = a.ctr[CTR_FRAME] & 1;

    // ---- stage the input (with its prologue)
    if (a.pro == PRO_RMSNORM) {
        // codec RMSNorm (qwen_codec.py:813-817): x * rsqrt(mean(x^2) + eps), then * weight; T == 1 here
        float ss = 0.f;
        for (int c = tid; c < Cin; c += blockDim.x) { float v = a.x[c * a.x_cs]; ss += v * v; }
        ss = block_sum(ss, red);
        float r = rsqrtf(ss / (float)Cin + a.eps);
        for (int c = tid; c < Cin; c += blockDim.x) xs[c] = (a.x[c * a.x_cs] * r) * a.p0[c];
    } else {
        for (int i = tid; i < Cin * T; i += blockDim.x) {
            int c = (KW == 1) ? i % Cin : i / T, t = (KW == 1) ? i / Cin : i % T;
            float v = a.x[c * a.x_cs + t * a.x_ts];
            if (a.pro == PRO_SNAKE) v = snake(v, a.p0[c], a.p1[c]);
            if (KW == 1) xs[t * Cin + c] = v; else xs[c * P + PAD + t] = v;
        }
        if constexpr (KW > 1) {
            const float* hist = a.state + parity * Cin * PAD;
            for (int i = tid; i < Cin * PAD; i += blockDim.x) xs[(i / PAD) * P + (i % PAD)] = hist[i];
        }
    }
    __syncthreads();
    if constexpr (KW > 1) if (blockIdx.x == 0) {
        // the next frame's history: the last PAD columns of [history | new]
        float* nxt = a.state + (parity ^ 1) * Cin * PAD;
        for (int i = tid; i < Cin * PAD; i += blockDim.x) nxt[i] = xs[(i / PAD) * P + T + (i % PAD)];
    }

    const int lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int Kd = Cin * KW;
    for (int row = blockIdx.x * nw + warp; row < a.rows; row += gridDim.x * nw) {
        const float4* wr = reinterpret_cast<const float4*>(a.w + (size_t)row * Kd);
        const float4* wr2 = DUAL ? reinterpret_cast<const float4*>(a.w2 + (size_t)row * Kd) : nullptr;
        float acc[T], acc2[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.f, acc2[t] = 0.f;
#pragma unroll 4
        for (int f4 = lane; f4 < Kd / 4; f4 += 32) {
            float4 w4 = __ldg(wr + f4);
            float4 u4 = DUAL ? __ldg(wr2 + f4) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float we[4] = {w4.x, w4.y, w4.z, w4.w};
            const float ue[4] = {u4.x, u4.y, u4.z, u4.w};
            if (KW == 1) {
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    float4 x4 = *reinterpret_cast<const float4*>(xs + t * Cin + f4 * 4);
                    acc[t] += we[0] * x4.x + we[1] * x4.y + we[2] * x4.z + we[3] * x4.w;
                    if (DUAL) acc2[t] += ue[0] * x4.x + ue[1] * x4.y + ue[2] * x4.z + ue[3] * x4.w;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int idx = f4 * 4 + e, ci = idx / KW, j = idx - ci * KW;
                    const float* xp = xs + ci * P + j;
#pragma unroll
                    for (int t = 0; t < T; ++t) acc[t] += we[e] * xp[t];
                }
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            acc[t] = warp_sum(acc[t]);
            if (DUAL) acc2[t] = warp_sum(acc2[t]);
        }
        if (lane == 0) {
            int g = row / a.row_div, r = row - g * a.row_div;
            float b = a.bias ? a.bias[g] : 0.f;
#pragma unroll
            for (int t = 0; t < T; ++t) {
                size_t o = (size_t)g * a.y_rs + (size_t)r * a.y_js + (size_t)t * a.y_ts;
                float v = acc[t] + b;
                if (a.epi == EPI_GELU) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
                else if (a.epi == EPI_SCALE_RES) v = a.res[o] + a.scale[g] * v;
                else if (a.epi == EPI_SILU_MUL) v = (v / (1.f + expf(-v))) * acc2[t];
                a.y[o] = v;
            }
        }
    }
}

// ---------------------------------------------------------------- transformer attention (one new position)
struct CAttnArgs {
    const float* qkv;     // [3 * H * 64] rows q | k | v of the new position (before RoPE)
    float* kc;            // [H][max_seq][64] keys of this layer (after RoPE)
    float* vc;            // [H][max_seq][64]
    const float* cos_t;   // [max_seq][64]
    const float* sin_t;
    float* out;           // [H * 64]
    int* ctr;
    int H, max_seq;
};

// DecTransformerBlock.forward, streaming branch (qwen_codec.py:948-964): RoPE (rotate-half), write K/V at the
// position, softmax(q K^T / 8) V over positions 0..pos.
__global__ void __launch_bounds__(128) k_ct_attn(CAttnArgs a) {
    __shared__ float q[64], sc[256], red[32], part[2][64];
    pdl_wait();
    pdl_launch();
    const int h = blockIdx.x, tid = threadIdx.x, HD = a.H * 64;
    int pos = a.ctr[CTR_POS];
    if (pos >= a.max_seq) {
        if (tid == 0 && h == 0) atomicOr(a.ctr + CTR_FLAG, FLAG_POS_OVERFLOW);
        pos = a.max_seq - 1;
    }
    float* kc = a.kc + (size_t)h * a.max_seq * 64;
    float* vc = a.vc + (size_t)h * a.max_seq * 64;
    if (tid < 64) {
        int i = tid, o = i < 32 ? i + 32 : i - 32;
        float c = a.cos_t[pos * 64 + i], s = a.sin_t[pos * 64 + i];
        float qi = a.qkv[h * 64 + i], qo = a.qkv[h * 64 + o];
        float ki = a.qkv[HD + h * 64 + i], ko = a.qkv[HD + h * 64 + o];
        q[i] = qi * c + (i < 32 ? -qo : qo) * s;
        kc[pos * 64 + i] = ki * c + (i < 32 ? -ko : ko) * s;
        vc[pos * 64 + i] = a.qkv[2 * HD + h * 64 + i];
    }
    __syncthreads();
    const int lane = tid & 31, warp = tid >> 5, n = pos + 1;
    for (int j = warp; j < n; j += 4) {
        float d = q[lane] * kc[j * 64 + lane] + q[lane + 32] * kc[j * 64 + lane + 32];
        d = warp_sum(d);
        if (lane == 0) sc[j] = d * 0.125f;
    }
    __syncthreads();
    float m = -INFINITY;
    for (int j = tid; j < n; j += 128) m = fmaxf(m, sc[j]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float s = 0.f;
    for (int j = tid; j < n; j += 128) { float e = expf(sc[j] - m); sc[j] = e; s += e; }
    s = block_sum(s, red);
    __syncthreads();
    const int d = tid & 63, half = tid >> 6;
    float acc = 0.f;
    for (int j = half; j < n; j += 2) acc += sc[j] * vc[j * 64 + d];
    part[half][d] = acc;
    __syncthreads();
    if (tid < 64) a.out[h * 64 + tid] = (part[0][tid] + part[1][tid]) / s;
}

// ---------------------------------------------------------------- ConvNeXt: depthwise conv + LayerNorm
struct DwLnArgs {
    const float* x;       // [C][T] channel-major
    const float* w;       // [C][7]
    const float* b;       // [C]
    const float* ln_w; const float* ln_b;
    float* state;         // [2][C * 6]
    const int* ctr;
    float* z;             // [T][C] time-major, normalised
    int C, T;
};

// ConvNeXtBlock.forward up to the LayerNorm (qwen_codec.py:841-846): causal depthwise k=7, LayerNorm over channels
__global__ void __launch_bounds__(256) k_dwconv_ln(DwLnArgs a) {
    __shared__ float red[32];
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x, tid = threadIdx.x, C = a.C, T = a.T;
    const int parity = a.ctr[CTR_FRAME] & 1;
    const float* hist = a.state + parity * C * 6;
    float v[4];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int c = tid + i * 256;
        float acc = 0.f;
        if (c < C) {
            acc = a.b[c];
#pragma unroll
            for (int j = 0; j < 7; ++j) {
                int p = t + j;   // index into [history(6) | new(T)]
                float xv = p < 6 ? hist[c * 6 + p] : a.x[c * T + (p - 6)];
                acc += a.w[c * 7 + j] * xv;
            }
            sum += acc;
        }
        v[i] = acc;
    }
    if (t == 0) {
        float* nxt = a.state + (parity ^ 1) * C * 6;
        for (int i = tid; i < C * 6; i += 256) {
            int c = i / 6, p = T + (i % 6);
            nxt[i] = p < 6 ? hist[c * 6 + p] : a.x[c * T + (p - 6)];
        }
    }
    float mean = block_sum(sum, red) / (float)C;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) if (tid + i * 256 < C) { float d = v[i] - mean; var += d * d; }
    var = block_sum(var, red) / (float)C;
    float r = rsqrtf(var + 1e-6f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int c = tid + i * 256;
        if (c < C) a.z[t * C + c] = (v[i] - mean) * r * a.ln_w[c] + a.ln_b[c];
    }
}

// ---------------------------------------------------------------- register-tiled convolution for long frames
struct TileArgs {
    const float* w;       // [Cout][Cin][KW]
    const float* bias;    // [Cout] or null
    const float* x;       // [Cin][T]
    float* state;         // [2][Cin * pad] activated history, or null when pad == 0
    const float* ea; const float* ib;   // SnakeBeta on the input, per input channel, or null
    const float* res;     // [Cout][T] residual or null
    float* y;             // [Cout][T]
    float* part;          // [splits][tiles][COT * 32] partial tiles
    int* tile_ctr;        // [tiles] arrival counters (zero between launches)
    const int* ctr;
    int Cin, Cout, T, dil, pad, splits, ci_per_split;
};

// y[co][t] = bias[co] + sum_{ci, j} w[co][ci][j] * act(X)[ci][t + j * dil - pad]   (+ res[co][t])
// grid (T / 32, ceil(Cout / COT), splits); 128 threads, each (COT / 16) x 4 outputs.
template <int KW, int COT>
__global__ void __launch_bounds__(128) k_ctile(TileArgs a) {
    constexpr int CC = 8;                       // input channels per staging step
    constexpr int CPT = COT / 16;               // output channels per thread
    constexpr int WS = CC * KW + 1;             // padded row stride of the weight tile
    constexpr int XW = 32 + (KW - 1) * 9;       // widest input window (dilation <= 9)
    __shared__ float ws[COT * WS];
    __shared__ float xw[CC * XW];
    __shared__ int s_last;
    pdl_wait();
    pdl_launch();
    const int tid = threadIdx.x, tx = tid & 7, ty = tid >> 3;
    const int t0 = blockIdx.x * 32, co0 = blockIdx.y * COT;
    const int Cin = a.Cin, T = a.T, dil = a.dil, pad = a.pad;
    const int win = 32 + (KW - 1) * dil;
    const int parity = a.ctr[CTR_FRAME] & 1;
    const float* hist = a.state ? a.state + (size_t)parity * Cin * pad : nullptr;
    const int ci_lo = blockIdx.z * a.ci_per_split, ci_hi = min(Cin, ci_lo + a.ci_per_split);

    // the next frame's history (last `pad` columns of [history | act(x)]), shared out over the whole grid
    if (a.state) {
        float* nxt = a.state + (size_t)(parity ^ 1) * Cin * pad;
        int nblk = gridDim.x * gridDim.y * gridDim.z;
        int blk = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        for (int i = blk * 128 + tid; i < Cin * pad; i += nblk * 128) {
            int c = i / pad, p = T + (i - c * pad);     // column in [history(pad) | new(T)]
            float v;
            if (p < pad) v = hist[c * pad + p];
            else {
                v = a.x[(size_t)c * T + (p - pad)];
                if (a.ea) v = snake(v, a.ea[c], a.ib[c]);
            }
            nxt[i] = v;
        }
    }

    float acc[CPT][4];
#pragma unroll
    for (int i = 0; i < CPT; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[i][k] = 0.f;

    for (int c0 = ci_lo; c0 < ci_hi; c0 += CC) {
        const int nc = min(CC, ci_hi - c0);
        for (int i = tid; i < COT * CC * KW; i += 128) {
            int r = i / (CC * KW), e = i - r * (CC * KW);
            int co = co0 + r;
            float v = 0.f;
            if (co < a.Cout && e < nc * KW) v = a.w[((size_t)co * Cin + c0) * KW + e];
            ws[r * WS + e] = v;
        }
        for (int i = tid; i < CC * win; i += 128) {
            int c = i / win, p = i - c * win;
            float v = 0.f;
            if (c < nc) {
                int ci = c0 + c, tt = t0 + p - pad;     // time index relative to this frame's first column
                if (tt < 0) { if (hist) v = hist[ci * pad + (pad + tt)]; }
                else if (tt < T) {
                    v = a.x[(size_t)ci * T + tt];
                    if (a.ea) v = snake(v, a.ea[ci], a.ib[ci]);
                }
            }
            xw[c * XW + p] = v;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < CC; ++c) {
#pragma unroll
            for (int j = 0; j < KW; ++j) {
                float wv[CPT], xv[4];
#pragma unroll
                for (int i = 0; i < CPT; ++i) wv[i] = ws[(ty * CPT + i) * WS + c * KW + j];
#pragma unroll
                for (int k = 0; k < 4; ++k) xv[k] = xw[c * XW + tx * 4 + k + j * dil];
#pragma unroll
                for (int i = 0; i < CPT; ++i)
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc[i][k] += wv[i] * xv[k];
            }
        }
        __syncthreads();
    }

    const int tile = blockIdx.y * gridDim.x + blockIdx.x, ntiles = gridDim.x * gridDim.y;
    if (a.splits > 1) {
        float* mine = a.part + ((size_t)blockIdx.z * ntiles + tile) * (COT * 32);
#pragma unroll
        for (int i = 0; i < CPT; ++i)
            *reinterpret_cast<float4*>(mine + (ty * CPT + i) * 32 + tx * 4) =
                make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int prev = atomicAdd(a.tile_ctr + tile, 1);
            s_last = (prev == a.splits - 1);
            if (s_last) a.tile_ctr[tile] = 0;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int i = 0; i < CPT; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[i][k] = 0.f;
        for (int s = 0; s < a.splits; ++s) {     // split order: the sum does not depend on arrival order
            const float* p = a.part + ((size_t)s * ntiles + tile) * (COT * 32);
#pragma unroll
            for (int i = 0; i < CPT; ++i) {
                float4 v = __ldcg(reinterpret_cast<const float4*>(p + (ty * CPT + i) * 32 + tx * 4));
                acc[i][0] += v.x; acc[i][1] += v.y; acc[i][2] += v.z; acc[i][3] += v.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        int co = co0 + ty * CPT + i;
        if (co >= a.Cout) continue;
        float b = a.bias ? a.bias[co] : 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int t = t0 + tx * 4 + k;
            if (t >= T) continue;
            float v = acc[i][k] + b;
            if (a.res) v += a.res[(size_t)co * T + t];
            a.y[(size_t)co * T + t] = v;
        }
    }
}

// ---------------------------------------------------------------- overlap-add of a transposed convolution
struct OlaArgs {
    const float* p;       // [(Cout * 2s)][Tin]: p[(co, k)][t] = sum_ci w[ci][co][k] * act(x)[ci][t]
    const float* bias;    // [Cout]
    float* partial;       // [Cout][s]: what the previous frame's last column adds to this frame's first s samples
    float* y;             // [Cout][Tin * s]
    int Cout, s, Tin;
};

// CausalTransConv1d.forward, streaming branch (qwen_codec.py:140-158) for kernel = 2 * stride
__global__ void __launch_bounds__(256) k_overlap_add(OlaArgs a) {
    pdl_wait();
    pdl_launch();
    const int s = a.s, Tin = a.Tin, K = 2 * s, Tout = Tin * s;
    int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= a.Cout * Tout) return;
    int co = i / Tout, u = i - co * Tout, t = u / s, j = u - t * s;
    float v = a.p[(size_t)(co * K + j) * Tin + t] + a.bias[co];
    if (t > 0) v += a.p[(size_t)(co * K + j + s) * Tin + t - 1];
    else {
        v += a.partial[co * s + j];
        a.partial[co * s + j] = a.p[(size_t)(co * K + j + s) * Tin + Tin - 1];   // read above by this thread only
    }
    a.y[i] = v;
}

// ---------------------------------------------------------------- last convolution (96 -> 1, k = 7) + clamp
struct FinalArgs {
    const float* x;       // [C][T]
    const float* w;       // [C][7]
    const float* bias;    // [1]
    const float* ea; const float* ib;
    float* state;         // [2][C * 6]
    const int* ctr;
    float* audio;         // [T]
    int C, T;
};

__global__ void __launch_bounds__(64) k_final_conv(FinalArgs a) {
    extern __shared__ float xs[];   // [C][70] activated window
    pdl_wait();
    pdl_launch();
    const int tid = threadIdx.x, t0 = blockIdx.x * 64, C = a.C, T = a.T;
    const int parity = a.ctr[CTR_FRAME] & 1;
    const float* hist = a.state + parity * C * 6;
    for (int i = tid; i < C * 70; i += 64) {
        int c = i / 70, p = i - c * 70, tt = t0 + p - 6;
        float v = 0.f;
        if (tt < 0) v = hist[c * 6 + 6 + tt];
        else if (tt < T) v = snake(a.x[c * T + tt], a.ea[c], a.ib[c]);
        xs[i] = v;
    }
    __syncthreads();
    if (blockIdx.x == gridDim.x - 1) {   // T >= 6: the new history is the last six activated columns
        float* nxt = a.state + (parity ^ 1) * C * 6;
        for (int i = tid; i < C * 6; i += 64) {
            int c = i / 6, p = i - c * 6;
            nxt[i] = xs[c * 70 + (T - t0) + p];
        }
    }
    int t = t0 + tid;
    if (t >= T) return;
    float acc = a.bias[0];
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int j = 0; j < 7; ++j) acc += a.w[c * 7 + j] * xs[c * 70 + tid + j];
    a.audio[t] = fminf(1.f, fmaxf(-1.f, acc));
}

// one frame done: advance the state parity and the transformer position
__global__ void k_advance(int* ctr) {
    pdl_wait();
    pdl_launch();
    if (threadIdx.x == 0) { ctr[CTR_FRAME] += 1; ctr[CTR_POS] += 1; }
}

}  // namespace vuic
