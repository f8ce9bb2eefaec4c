// Codec encoder (24 kHz audio -> 16 codebook indices per 80 ms frame), fp32: the device work of the reference's
// QwenCodecEncoder.forward (src/vui/qwen_codec.py:385-390) as StreamingCodecEncoder drives it over a fixed 10 s
// buffer (671-805): causal convolution stack with ELU and strides 4, 5, 6, 8 (278-311), an 8-layer causal
// transformer over 25 Hz frames with LayerNorm, rotate-half RoPE, GELU MLP and per-channel layer scales (314-365),
// a stride-2 convolution to 12.5 Hz, and split residual vector quantisation: nearest code of 2048, residual
// subtracted, next codebook (185-275).
//
// Activations are channel-major [C][T] like torch's (1, C, T).  One tiled kernel does every convolution and every
// linear layer (a k = 1 convolution): 32 output channels x 64 columns per CTA, input windows and weight slabs
// staged in shared memory, ELU applied while staging, epilogues bias / GELU / layer-scale + residual.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vuie {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

enum { EE_BIAS = 0, EE_GELU = 1, EE_SCALE_RES = 2, EE_RES = 3 };

struct EConvArgs {
    const float* w;      // [Cout][Cin][K] (torch layout)
    const float* bias;   // [Cout] or null
    const float* x;      // [Cin][Tin]
    const float* res;    // [Cout][Tout] (EE_SCALE_RES, EE_RES)
    const float* scale;  // [Cout] (EE_SCALE_RES)
    float* y;            // [Cout][Tout]
    int Cin, Cout, K, stride, Tin, Tout;
    int cc;              // input channels per staging step (8, or 32 for k = 1: fewer, fatter steps)
    int elu_in;          // ELU on the input (the nn.ELU() that precedes the convolution)
    int epi;
};

constexpr int EC_CO = 32, EC_T = 64, EC_THREADS = 128;

// y[co][t] = bias[co] + sum_{ci, j} w[co][ci][j] * act(x)[ci][t * stride + j - (K - stride)]   (zero left padding:
// CausalConv1d outside a streaming context, qwen_codec.py:92-98), then the epilogue.
// grid (ceil(Tout / 64), ceil(Cout / 32)); 128 threads, each 4 output channels x 8 columns (t = tx + 8 k).
__global__ void __launch_bounds__(EC_THREADS) k_econv(EConvArgs a) {
    extern __shared__ float sm[];
    const int K = a.K, s = a.stride, pad = K - s;
    const int XW = EC_T * s + pad;                 // input columns one tile needs
    const int CC = a.cc;
    float* xs = sm;                                // [CC][XW]
    float* ws = sm + CC * XW;                      // [32][CC * K + 1]
    const int WS = CC * K + 1;
    const int tid = threadIdx.x, tx = tid & 7, ty = tid >> 3;   // ty: 16 groups of 2 channels
    const int t0 = blockIdx.x * EC_T, co0 = blockIdx.y * EC_CO;
    const int x0 = t0 * s - pad;                   // input column of window position 0
    float acc[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
    for (int c0 = 0; c0 < a.Cin; c0 += CC) {
        const int nc = min(CC, a.Cin - c0);
        // staging loads are unrolled so that several are in flight (they are what bounds a step at small grids)
#pragma unroll 8
        for (int i = tid; i < CC * XW; i += EC_THREADS) {
            const int c = i / XW, p = i - c * XW, col = x0 + p;
            float v = 0.f;
            if (c < nc && col >= 0 && col < a.Tin) {
                v = __ldg(a.x + (size_t)(c0 + c) * a.Tin + col);
                if (a.elu_in) v = v > 0.f ? v : expm1f(v);
            }
            xs[i] = v;
        }
#pragma unroll 8
        for (int i = tid; i < EC_CO * CC * K; i += EC_THREADS) {
            const int r = i / (CC * K), e = i - r * (CC * K), co = co0 + r;
            float v = 0.f;
            if (co < a.Cout && e < nc * K) v = __ldg(a.w + ((size_t)co * a.Cin + c0) * K + e);
            ws[r * WS + e] = v;
        }
        __syncthreads();
#pragma unroll 2
        for (int c = 0; c < nc; ++c)
            for (int j = 0; j < K; ++j) {
                const float w0 = ws[(ty * 2) * WS + c * K + j], w1 = ws[(ty * 2 + 1) * WS + c * K + j];
                const float* xr = xs + c * XW + j;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float xv = xr[(tx + 8 * k) * s];
                    acc[0][k] += w0 * xv;
                    acc[1][k] += w1 * xv;
                }
            }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int co = co0 + ty * 2 + i;
        if (co >= a.Cout) continue;
        const float b = a.bias ? __ldg(a.bias + co) : 0.f;
        const float sc = a.epi == EE_SCALE_RES ? __ldg(a.scale + co) : 1.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int t = t0 + tx + 8 * k;
            if (t >= a.Tout) continue;
            float v = acc[i][k] + b;
            const size_t o = (size_t)co * a.Tout + t;
            if (a.epi == EE_GELU) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
            else if (a.epi == EE_SCALE_RES) v = a.res[o] + sc * v;
            else if (a.epi == EE_RES) v = a.res[o] + v;
            a.y[o] = v;
        }
    }
}

// LayerNorm over channels (eps 1e-5, weight and bias) for every column of x [C][T] -> y [C][T].
// One warp per column pair would waste loads; a CTA takes 32 columns: thread (g, l) sums channels g, g + 8, ... of
// column l, the 8 groups meet in shared memory.
__global__ void __launch_bounds__(256) k_elayernorm(const float* x, const float* w, const float* b, float* y, int C, int T) {
    __shared__ float s1[8][32], s2[8][32];
    const int l = threadIdx.x & 31, g = threadIdx.x >> 5, t = blockIdx.x * 32 + l;
    float sum = 0.f;
    if (t < T)
        for (int c = g; c < C; c += 8) sum += x[(size_t)c * T + t];
    s1[g][l] = sum;
    __syncthreads();
    float mean = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) mean += s1[i][l];
    mean /= (float)C;
    float var = 0.f;
    if (t < T)
        for (int c = g; c < C; c += 8) { const float d = x[(size_t)c * T + t] - mean; var += d * d; }
    s2[g][l] = var;
    __syncthreads();
    var = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) var += s2[i][l];
    const float r = rsqrtf(var / (float)C + 1e-5f);
    if (t < T)
        for (int c = g; c < C; c += 8) y[(size_t)c * T + t] = (x[(size_t)c * T + t] - mean) * r * w[c] + b[c];
}

// Causal attention with rotate-half RoPE (EncTransformerBlock.forward, qwen_codec.py:332-345): q, k, v are
// [H * 64][T]; one warp per (head, query), lane l holds dimensions l and l + 32 (a rotate-half pair); online softmax.
__global__ void __launch_bounds__(128) k_eattn(const float* q, const float* k, const float* v, const float* cos_t,
                                               const float* sin_t, float* out, int H, int T) {
    const int lane = threadIdx.x & 31, w = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= H * T) return;
    const int h = w / T, t = w - h * T;
    const size_t r0 = (size_t)(h * 64 + lane) * T, r1 = (size_t)(h * 64 + lane + 32) * T;
    const float c0 = cos_t[t * 64 + lane], s0 = sin_t[t * 64 + lane];
    const float c1 = cos_t[t * 64 + lane + 32], s1 = sin_t[t * 64 + lane + 32];
    const float qa = q[r0 + t], qb = q[r1 + t];
    const float q0 = qa * c0 - qb * s0, q1 = qb * c1 + qa * s1;
    float m = -INFINITY, lsum = 0.f, a0 = 0.f, a1 = 0.f;
    for (int j = 0; j <= t; ++j) {
        const float ka = k[r0 + j], kb = k[r1 + j];
        const float kc0 = cos_t[j * 64 + lane], ks0 = sin_t[j * 64 + lane];
        const float kc1 = cos_t[j * 64 + lane + 32], ks1 = sin_t[j * 64 + lane + 32];
        float d = q0 * (ka * kc0 - kb * ks0) + q1 * (kb * kc1 + ka * ks1);
        d = warp_sum(d) * 0.125f;
        const float mn = fmaxf(m, d), corr = expf(m - mn), p = expf(d - mn);
        lsum = lsum * corr + p;
        a0 = a0 * corr + p * v[r0 + j];
        a1 = a1 * corr + p * v[r1 + j];
        m = mn;
    }
    out[r0 + t] = a0 / lsum;
    out[r1 + t] = a1 / lsum;
}

// Residual vector quantisation of one frame per CTA (ResidualVQ.encode / EuclideanCodebook.encode,
// qwen_codec.py:190-195, 218-229): for each codebook the nearest of 2048 codes (first index on ties, as argmin),
// then the residual loses that code.  torch.cdist's distances are sqrt(|x|^2 + |e|^2 - 2 x.e) for inputs of this
// size; the argmin of |e|^2 - 2 x.e is the same.
struct ERvqArgs {
    const float* h;          // [256][T] projected latents of this quantiser group
    const float* table[16];  // codebooks (2048, 256)
    const float* norm2[16];  // |e|^2 per code (2048)
    long long* codes;        // [n_total][T]; this group writes rows q0 .. q0 + n - 1
    int n, q0, T;
};

__global__ void __launch_bounds__(256) k_ervq(ERvqArgs a) {
    __shared__ float r[256];
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    __shared__ int pick;
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    r[tid] = a.h[(size_t)tid * a.T + t];
    __syncthreads();
    for (int cb = 0; cb < a.n; ++cb) {
        const float* E = a.table[cb];
        float rv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) rv[j] = r[lane * 8 + j];
        float bv = INFINITY;
        int bi = 0;
        for (int c = warp; c < 2048; c += 8) {      // a warp reads a code's 1 KB row at once
            const float4 e0 = __ldg(reinterpret_cast<const float4*>(E + (size_t)c * 256 + lane * 8));
            const float4 e1 = __ldg(reinterpret_cast<const float4*>(E + (size_t)c * 256 + lane * 8 + 4));
            float d = rv[0] * e0.x + rv[1] * e0.y + rv[2] * e0.z + rv[3] * e0.w + rv[4] * e1.x + rv[5] * e1.y +
                      rv[6] * e1.z + rv[7] * e1.w;
            d = warp_sum(d);
            const float dist = __ldg(a.norm2[cb] + c) - 2.f * d;
            if (dist < bv) { bv = dist; bi = c; }    // c ascends: the first minimum is kept
        }
        if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
            float v0 = best_v[0];
            int i0 = best_i[0];
            for (int i = 1; i < 8; ++i)
                if (best_v[i] < v0 || (best_v[i] == v0 && best_i[i] < i0)) { v0 = best_v[i]; i0 = best_i[i]; }
            pick = i0;
            a.codes[(size_t)(a.q0 + cb) * a.T + t] = i0;
        }
        __syncthreads();
        r[tid] -= __ldg(E + (size_t)pick * 256 + tid);
        __syncthreads();
    }
}

}  // namespace vuie
