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
//   k_ctile : register-tiled (co x t) convolution with dilation for the long stages: a cp.async
//             ring of K-major weight slabs and input windows, K split over CTAs with an ordered
//             last-arriver reduction; its input was activated (SnakeBeta) by the producing kernel.
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
constexpr int FLAG_WAIT = 4;        // a bounded wait on an asynchronous copy ran out

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
    long long code[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) code[q] = q < a.n_q ? a.codes[q] : 0;
    bool bad = false;
#pragma unroll
    for (int q = 0; q < 16; ++q)
        if (code[q] < 0 || code[q] >= 2048) { bad = true; code[q] = code[q] < 0 ? 0 : 2047; }
    if (bad && c == 0) atomicOr(a.ctr + CTR_FLAG, FLAG_BAD_CODE);
    float v[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) v[q] = q < a.n_q ? __ldg(a.table[q] + code[q] * 256 + c) : 0.f;
    float sem = v[0], acq = 0.f;
#pragma unroll
    for (int q = 1; q < 16; ++q) acq += v[q];     // codebook order, as the reference's running sum
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
    int ksplit;           // warps that share one row: 1, 2, 4 or 8 (Cin * KW / 4 divisible by 32 * ksplit)
    int pro;              // PRO_*
    const float* p0;      // RMSNorm weight | snake ea
    const float* p1;      // snake ib
    float eps;
    int epi;              // EPI_*
    float* y;             // output (row, t) at y[(row / row_div) * y_rs + (row % row_div) * y_js + t * y_ts]
    int row_div, y_rs, y_js, y_ts;
    const float* scale;   // EPI_SCALE_RES: per-(row / row_div) factor
    const float* res;     // EPI_SCALE_RES: residual, indexed like y
    float* y_act;         // optional: snake(v) with the consumer's per-row parameters, indexed like y
    const float* act_ea; const float* act_ib;
};

// out[row][t] = sum_{ci, j} w[row][ci][j] * X[ci][t + j]  with X = [history | new columns] (causal, dilation 1)
template <int KW, int T, bool DUAL>
__global__ void __launch_bounds__(256) k_crows(RowsArgs a) {
    extern __shared__ float xs[];   // KW == 1: [T][Cin];  KW > 1: [Cin][P], P = KW - 1 + T
    __shared__ float red[32];
    __shared__ float ksum[8][2 * T];
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
    } else if (KW == 1 && a.x_cs == 1 && a.pro == PRO_NONE) {
        // time-major input: every column is a contiguous run of Cin floats
        for (int t = 0; t < T; ++t) {
            const float4* src = reinterpret_cast<const float4*>(a.x + (size_t)t * a.x_ts);
            float4* dst = reinterpret_cast<float4*>(xs + t * Cin);
#pragma unroll 8
            for (int i = tid; i < Cin / 4; i += blockDim.x) dst[i] = __ldg(src + i);
        }
    } else {
#pragma unroll 8
        for (int i = tid; i < Cin * T; i += blockDim.x) {
            int c = (KW == 1) ? i % Cin : i / T, t = (KW == 1) ? i / Cin : i % T;
            float v = __ldg(a.x + c * a.x_cs + t * a.x_ts);
            if (a.pro == PRO_SNAKE) v = snake(v, __ldg(a.p0 + c), __ldg(a.p1 + c));
            if (KW == 1) xs[t * Cin + c] = v; else xs[c * P + PAD + t] = v;
        }
        if constexpr (KW > 1) {
            const float* hist = a.state + parity * Cin * PAD;
#pragma unroll 8
            for (int i = tid; i < Cin * PAD; i += blockDim.x) xs[(i / PAD) * P + (i % PAD)] = __ldg(hist + i);
        }
    }
    __syncthreads();
    if constexpr (KW > 1) if (blockIdx.x == 0) {
        // the next frame's history: the last PAD columns of [history | new]
        float* nxt = a.state + (parity ^ 1) * Cin * PAD;
        for (int i = tid; i < Cin * PAD; i += blockDim.x) nxt[i] = xs[(i / PAD) * P + T + (i % PAD)];
    }

    // S warps share a row (each a contiguous 1/S of K), 8 / S rows per pass; partial sums meet in shared memory
    // and are added in warp order, so the result does not depend on timing.
    const int lane = tid & 31, warp = tid >> 5;
    const int S = a.ksplit, rpp = 8 / S, sub = warp % S;
    const int Kd = Cin * KW, per4 = Kd / 4 / S;
    for (int rowbase = blockIdx.x * rpp; rowbase < a.rows; rowbase += gridDim.x * rpp) {
        const int row = rowbase + warp / S;
        float acc[T], acc2[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.f, acc2[t] = 0.f;
        if (row < a.rows) {
            const float4* wr = reinterpret_cast<const float4*>(a.w + (size_t)row * Kd) + sub * per4;
            const float4* wr2 = DUAL ? reinterpret_cast<const float4*>(a.w2 + (size_t)row * Kd) + sub * per4 : nullptr;
#pragma unroll 8
            for (int f4 = lane; f4 < per4; f4 += 32) {
                float4 w4 = __ldg(wr + f4);
                float4 u4 = DUAL ? __ldg(wr2 + f4) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float we[4] = {w4.x, w4.y, w4.z, w4.w};
                const float ue[4] = {u4.x, u4.y, u4.z, u4.w};
                const int g4 = sub * per4 + f4;
                if (KW == 1) {
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        float4 x4 = *reinterpret_cast<const float4*>(xs + t * Cin + g4 * 4);
                        acc[t] += we[0] * x4.x + we[1] * x4.y + we[2] * x4.z + we[3] * x4.w;
                        if (DUAL) acc2[t] += ue[0] * x4.x + ue[1] * x4.y + ue[2] * x4.z + ue[3] * x4.w;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        int idx = g4 * 4 + e, ci = idx / KW, j = idx - ci * KW;
                        const float* xp = xs + ci * P + j;
#pragma unroll
                        for (int t = 0; t < T; ++t) acc[t] += we[e] * xp[t];
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            acc[t] = warp_sum(acc[t]);
            if (DUAL) acc2[t] = warp_sum(acc2[t]);
        }
        if (S > 1) {
            __syncthreads();
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < T; ++t) { ksum[warp][t] = acc[t]; if (DUAL) ksum[warp][T + t] = acc2[t]; }
            }
            __syncthreads();
            if (lane == 0 && sub == 0) {
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    acc[t] = 0.f; acc2[t] = 0.f;
                    for (int q = 0; q < S; ++q) { acc[t] += ksum[warp + q][t]; if (DUAL) acc2[t] += ksum[warp + q][T + t]; }
                }
            }
        }
        if (lane == 0 && sub == 0 && row < a.rows) {
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
                if (a.y_act) a.y_act[o] = snake(v, a.act_ea[g], a.act_ib[g]);
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
// Activations that feed a convolution are stored ALREADY ACTIVATED by their producer (SnakeBeta applied once
// per element, in the producer's epilogue), in a buffer the convolution can copy from without arithmetic:
//   k = 1 : plain [C][T];
//   k = 7 : [2 parities][C][ld] with the P = 6 * dilation history columns in front: column c < P is history,
//           column P + t is this frame's t.  The frame of parity p reads buffer p; the convolution itself copies
//           its last P columns into the history columns of buffer p ^ 1 for the next frame.
struct ActOut {           // optional second output of a producer: snake(v) into a consumer's input buffer
    float* base;          // parity-0 buffer (null: none)
    long long pstride;    // elements between the two parity buffers (0: not double-buffered)
    int ld, off;          // element (co, t) at base[parity * pstride + co * ld + off + t]
    const float* ea; const float* ib;
};

__device__ __forceinline__ void act_store(const ActOut& o, int parity, int co, int t, float v) {
    if (o.base) o.base[(size_t)parity * o.pstride + (size_t)co * o.ld + o.off + t] = snake(v, o.ea[co], o.ib[co]);
}

struct TileArgs {
    const float* wt;      // weights per 96-channel output tile, K-major inside: [Cout / 96][Cin][KW][96]
    const float* bias;    // [Cout] or null
    const float* xa;      // activated input, parity-0 buffer
    long long x_pstride;  // elements between the parity buffers (0 when P == 0)
    int x_ld, P;          // row stride; history columns (KW - 1) * dil
    const float* res;     // [Cout][T] residual or null
    float* y;             // [Cout][T] plain output or null
    ActOut act;
    float* part;          // [splits][tiles][96 * 32] partial tiles
    int* tile_ctr;        // [tiles] arrival counters (zero between launches)
    const int* ctr;
    int Cin, Cout, T, dil, splits, ci_per_split;
};

// ---- bulk asynchronous copies counted on an mbarrier (no multicast), bounded waits
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, unsigned limit) {
    const uint32_t a = smem_u32(bar);
    for (unsigned spins = 0; spins < limit; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
// this thread's earlier cp.async copies count as one arrival on `bar` once they have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

#ifdef VUIC_TRACE
__device__ long long g_ct_trace[16];
#define CT_STAMP(n) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) g_ct_trace[n] = clock64(); } while (0)
#else
#define CT_STAMP(n) do {} while (0)
#endif

constexpr int CT_CO = 96, CT_T = 32, CT_GROUPS = 4, CT_THREADS = 96 * CT_GROUPS, CT_STAGES = 4;
constexpr unsigned CT_WAIT_LIMIT = 1u << 22;
template <int KW> struct CtCfg {
    static constexpr int CC = KW == 1 ? 32 : 8;                      // input channels per staging step
    static constexpr int XW = (32 + (KW - 1) * 9 + 3) / 4 * 4;       // widest input window (dilation <= 9)
};
template <int KW> constexpr int ct_smem_bytes() {
    return CT_STAGES * (CtCfg<KW>::CC * KW * CT_CO + CtCfg<KW>::CC * CtCfg<KW>::XW) * 4;
}

// y[co][t] = bias[co] + sum_{ci, j} w[ci][j][co] * xa[ci][t + j * dil]  (+ res[co][t]), xa as described above.
// Weights are stored per 96-channel output tile, K-major inside it: wt[co / 96][ci][j][co % 96], so the slab of
// one staging step (CC input channels) is one contiguous run.
// grid (T / 32, Cout / 96, splits); 384 threads = four groups of 96, each thread 8 output channels x 4 columns
// (t = tx + 8 k); the groups take every fourth input channel of a staging step and add up at the end: twelve
// warps per tile, three per scheduler, so shared-memory latency hides behind other warps' FMAs.
// The launch is a chain of memory round trips around little arithmetic, so each is started as early as it can be:
// thread 0 requests the first four weight slabs (one bulk copy each) before the dependency wait, all threads the
// input windows right after it (16-byte cp.async pieces that arrive on the same mbarrier), and a stage is refilled
// as soon as it has been consumed; partial tiles and outputs move as whole rows.  Waits on the copies are bounded
// and set FLAG_WAIT instead of hanging.
template <int KW>
__global__ void __launch_bounds__(CT_THREADS, 2) k_ctile(TileArgs a) {
    constexpr int CC = CtCfg<KW>::CC, XW = CtCfg<KW>::XW, KK = CC * KW, NST = CT_STAGES;
    constexpr int WST = KK * CT_CO, XST = CC * XW, SST = WST + XST;
    extern __shared__ __align__(128) float sm[];        // [stages][weight slab | input windows]
    __shared__ __align__(8) uint64_t full[NST];
    __shared__ int s_last;
    const int tid = threadIdx.x, grp = tid / 96, lt = tid - grp * 96, tx = lt & 7, ty = lt >> 3;
    const int lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.x * CT_T, co0 = blockIdx.y * CT_CO;
    const int Cin = a.Cin, T = a.T, dil = a.dil, P = a.P;
    const int ci_lo = blockIdx.z * a.ci_per_split, ci_hi = min(Cin, ci_lo + a.ci_per_split);
    const int nchunks = (ci_hi - ci_lo) / CC;
    const int win4 = (CT_T + P + 3) / 4;                // 16-byte pieces of one input window
    const float* wt = a.wt + (size_t)blockIdx.y * Cin * KW * CT_CO;
    CT_STAMP(0);
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < NST; ++s) mbar_init(&full[s], 1 + CT_THREADS);   // thread 0's expect_tx + everyone's windows
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    auto arm_and_load_w = [&](int st, int ch) {         // thread 0
        mbar_expect_tx(&full[st], WST * 4);
        bulk_g2s(sm + st * SST, wt + (size_t)(ci_lo + ch * CC) * KW * CT_CO, WST * 4, &full[st]);
    };
    if (tid == 0)
        for (int s = 0; s < NST && s < nchunks; ++s) arm_and_load_w(s, s);
    pdl_wait();
    pdl_launch();
    const int parity = a.ctr[CTR_FRAME] & 1;
    CT_STAMP(1);
    const float* xa = a.xa + (size_t)parity * a.x_pstride;
    auto load_x = [&](int st, int ch) {                 // all threads: piece q of channel c's window
        for (int i = tid; i < CC * win4; i += CT_THREADS) {
            const int c = i / win4, q = i - c * win4;
            cp_async16(sm + st * SST + WST + c * XW + q * 4, xa + (size_t)(ci_lo + ch * CC + c) * a.x_ld + t0 + q * 4);
        }
        cp_async_arrive(&full[st]);
    };
    for (int s = 0; s < NST && s < nchunks; ++s) load_x(s, s);

    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[i][k] = 0.f;

    CT_STAMP(2);
    constexpr int NIT = (CC / CT_GROUPS) * KW;          // (channel, tap) steps of one group per staging step
    for (int ch = 0; ch < nchunks; ++ch) {
        const int st = ch % NST;
        if (!mbar_wait(&full[st], (ch / NST) & 1, CT_WAIT_LIMIT) && lt == 0)
            atomicOr(const_cast<int*>(a.ctr) + CTR_FLAG, FLAG_WAIT);
        if (ch < 4) CT_STAMP(3 + ch);
        const float* w = sm + st * SST + grp * (KW * CT_CO) + ty * 8;
        const float* x = sm + st * SST + WST + grp * XW + tx;
        // operands of step it + 1 are requested before the FMAs of step it
        float4 a0 = *reinterpret_cast<const float4*>(w), a1 = *reinterpret_cast<const float4*>(w + 4);
        float bv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) bv[k] = x[8 * k];
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
            float4 n0 = a0, n1 = a1;
            float nb[4] = {0.f, 0.f, 0.f, 0.f};
            if (it + 1 < NIT) {
                const int cc = (it + 1) / KW, j = (it + 1) - cc * KW;
                const float* wn = w + (cc * CT_GROUPS * KW + j) * CT_CO;
                n0 = *reinterpret_cast<const float4*>(wn);
                n1 = *reinterpret_cast<const float4*>(wn + 4);
#pragma unroll
                for (int k = 0; k < 4; ++k) nb[k] = x[cc * CT_GROUPS * XW + 8 * k + j * dil];
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[0][k] += a0.x * bv[k]; acc[1][k] += a0.y * bv[k];
                acc[2][k] += a0.z * bv[k]; acc[3][k] += a0.w * bv[k];
                acc[4][k] += a1.x * bv[k]; acc[5][k] += a1.y * bv[k];
                acc[6][k] += a1.z * bv[k]; acc[7][k] += a1.w * bv[k];
            }
            a0 = n0; a1 = n1;
#pragma unroll
            for (int k = 0; k < 4; ++k) bv[k] = nb[k];
        }
        __syncthreads();                                 // the stage has been read by everyone: refill it
        if (ch + NST < nchunks) {
            if (tid == 0) arm_and_load_w(st, ch + NST);
            load_x(st, ch + NST);
        }
    }
    CT_STAMP(7);
    // the groups' sums meet in the (now idle) staging memory; groups 1..3 park theirs element-major (element e of
    // thread lt at [e][lt]: no bank conflicts), group 0 adds in group order and lays the tile out by rows
    float* const tl = sm;                                // final tile [96][TLS]
    constexpr int TLS = CT_T + 1, TL = CT_CO * CT_T;
    float* const park = sm + CT_CO * TLS;                // [3][32][96]
    if (grp > 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) park[((grp - 1) * 32 + i * 4 + k) * 96 + lt] = acc[i][k];
    }
    __syncthreads();
    if (grp > 0 && P > 0) {
        // meanwhile the other groups copy the next frame's history: my last P columns into the other parity's first P
        float* nxt = const_cast<float*>(a.xa) + (size_t)(parity ^ 1) * a.x_pstride;
        const int nthr = gridDim.x * gridDim.y * gridDim.z * (CT_THREADS - 96);
        const int me = ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * (CT_THREADS - 96) + (tid - 96);
        for (int i0 = me; i0 < Cin * P; i0 += 4 * nthr) {
            float hv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                int i = i0 + u * nthr, c = i / P, p = i - c * P;
                hv[u] = i < Cin * P ? xa[(size_t)c * a.x_ld + T + p] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                int i = i0 + u * nthr, c = i / P, p = i - c * P;
                if (i < Cin * P) nxt[(size_t)c * a.x_ld + p] = hv[u];
            }
        }
    }
    if (grp == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int e = (i * 4 + k) * 96 + lt;
                tl[(ty * 8 + i) * TLS + tx + 8 * k] = ((acc[i][k] + park[e]) + park[32 * 96 + e]) + park[2 * 32 * 96 + e];
            }
    }
    __syncthreads();
    CT_STAMP(8);

    const int tile = blockIdx.y * gridDim.x + blockIdx.x, ntiles = gridDim.x * gridDim.y;
    constexpr int EPT = TL / CT_THREADS;                 // tile elements per thread (8), lane = column
    if (a.splits > 1) {
        float* mine = a.part + ((size_t)blockIdx.z * ntiles + tile) * TL;
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * CT_THREADS;
            mine[e] = tl[(e >> 5) * TLS + (e & 31)];
        }
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
        float sum[EPT];
#pragma unroll
        for (int u = 0; u < EPT; ++u) sum[u] = 0.f;
#pragma unroll 4
        for (int s = 0; s < a.splits; ++s) {     // split order: the sum does not depend on arrival order
            const float* p = a.part + ((size_t)s * ntiles + tile) * TL;
#pragma unroll
            for (int u = 0; u < EPT; ++u) sum[u] += __ldcg(p + tid + u * CT_THREADS);
        }
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * CT_THREADS;
            tl[(e >> 5) * TLS + (e & 31)] = sum[u];
        }
        __syncthreads();
    }

    // epilogue by rows: warp w owns 8 output channels, lane = column; operands first, then the stores
    const int t = t0 + lane;
    constexpr int RPW = CT_CO / (CT_THREADS / 32);
    float bv2[RPW], ea[RPW], ib[RPW], rv[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int co = co0 + warp * RPW + r;
        bv2[r] = a.bias ? __ldg(a.bias + co) : 0.f;
        ea[r] = a.act.base ? __ldg(a.act.ea + co) : 0.f;
        ib[r] = a.act.base ? __ldg(a.act.ib + co) : 0.f;
        rv[r] = (a.res && t < T) ? a.res[(size_t)co * T + t] : 0.f;
    }
    float* act_dst = a.act.base ? a.act.base + (size_t)parity * a.act.pstride + a.act.off : nullptr;
    CT_STAMP(9);
    if (t < T) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int col = warp * RPW + r, co = co0 + col;
            float v = tl[col * TLS + lane] + bv2[r] + rv[r];
            if (a.y) a.y[(size_t)co * T + t] = v;
            if (act_dst) act_dst[(size_t)co * a.act.ld + t] = snake(v, ea[r], ib[r]);
        }
    }
    CT_STAMP(10);
}

// ---------------------------------------------------------------- overlap-add of a transposed convolution
struct OlaArgs {
    const float* p;       // [(Cout * 2s)][Tin]: p[(co, k)][t] = sum_ci w[ci][co][k] * act(x)[ci][t]
    const float* bias;    // [Cout]
    float* partial;       // [Cout][s]: what the previous frame's last column adds to this frame's first s samples
    float* y;             // [Cout][Tin * s]
    ActOut act;           // activated copy for the first residual unit
    const int* ctr;
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
    act_store(a.act, a.ctr[CTR_FRAME] & 1, co, u, v);
}

// ---------------------------------------------------------------- last convolution (96 -> 1, k = 7) + clamp
struct FinalArgs {
    const float* xa;      // activated input [2][C][ld] with 6 history columns in front (as for k_ctile)
    long long x_pstride; int x_ld;
    const float* w;       // [C][7]
    const float* bias;    // [1]
    const int* ctr;
    float* audio;         // [T]
    int C, T;
};

// 32 outputs per CTA; the CTA's input window (C x 38) goes to shared memory with every load in flight, then four
// groups of threads each sum a quarter of the channels
__global__ void __launch_bounds__(128) k_final_conv(FinalArgs a) {
    extern __shared__ float win[];       // [C][40]
    __shared__ float part[4][32];
    pdl_wait();
    pdl_launch();
    const int tid = threadIdx.x, lane = tid & 31, grp = tid >> 5, C = a.C, T = a.T;
    const int parity = a.ctr[CTR_FRAME] & 1;
    const float* xa = a.xa + (size_t)parity * a.x_pstride;
    const int t0 = blockIdx.x * 32;
#pragma unroll 8
    for (int i = tid; i < C * 10; i += 128) {      // 10 float4 pieces per channel: columns t0 .. t0 + 39
        const int c = i / 10, q = i - c * 10;
        reinterpret_cast<float4*>(win)[i] = *reinterpret_cast<const float4*>(xa + (size_t)c * a.x_ld + t0 + q * 4);
    }
    if (blockIdx.x == 0) {
        float* nxt = const_cast<float*>(a.xa) + (size_t)(parity ^ 1) * a.x_pstride;
        for (int i = tid; i < C * 6; i += 128) {
            int c = i / 6, p = i - c * 6;
            nxt[(size_t)c * a.x_ld + p] = xa[(size_t)c * a.x_ld + T + p];
        }
    }
    __syncthreads();
    const int t = t0 + lane, per = (C + 3) / 4;
    float acc = 0.f;
    const int c_lo = grp * per, c_hi = min(C, (grp + 1) * per);
#pragma unroll 4
    for (int c = c_lo; c < c_hi; ++c) {
        const float* xr = win + c * 40 + lane;
#pragma unroll
        for (int j = 0; j < 7; ++j) acc += __ldg(a.w + c * 7 + j) * xr[j];
    }
    part[grp][lane] = acc;
    __syncthreads();
    if (grp == 0 && t < T) {
        float v = a.bias[0] + ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane]));
        a.audio[t] = fminf(1.f, fmaxf(-1.f, v));
    }
}

// one frame done: advance the state parity and the transformer position
__global__ void k_advance(int* ctr) {
    pdl_wait();
    pdl_launch();
    if (threadIdx.x == 0) { ctr[CTR_FRAME] += 1; ctr[CTR_POS] += 1; }
}

}  // namespace vuic
