// Device code for the Vui Nano decode step on sm_100a: weight-streaming batched
// GEMV with fused RMSNorm / RoPE / KV-append / SwiGLU / residual epilogues,
// ragged split-KV GQA decode attention, the depth-transformer attention, and the
// per-codebook sampler.
//
// Numerics follow the reference's bf16 rounding points (src/vui/model.py 286-297,
// 204-258, 261-283; src/vui/rope.py 50): every tensor PyTorch materialises in
// bf16 is rounded to bf16 here at the same place; GEMV sums are fp32.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vuib {

typedef __nv_bfloat16 bf16;

constexpr int HD = 64;             // head_dim of backbone and depth transformer
constexpr int GEMV_THREADS = 256;  // 8 warps; one work item (1-2 weight rows) per warp
constexpr int GEMV_WARPS = 8;
constexpr int ATT_SPLIT = 128;     // keys per CTA in the backbone attention
constexpr int ATT_THREADS = 128;
constexpr int ATT_ITERS = ATT_SPLIT / 16;  // 4 warps x 4 key groups per pass
constexpr int PART_STRIDE = HD + 2;        // acc[64], m, l
constexpr int SAMPLE_THREADS = 256;
constexpr int SAMPLE_EL = 8;               // codebook_size = 256 * 8
constexpr int REP_HIST_MAX = 64;

enum DeviceFlag { FLAG_BAD_SLOT = 1, FLAG_BAD_POS = 2, FLAG_BAD_CODE = 4 };

// Device-side control block (lives in the workspace; vuib_set_sampling fills it).
struct SamplingCtl {
    float temperature;
    int32_t top_k_cb0;
    int32_t top_k_rq;
    float rep_penalty;
    int32_t rep_window;
    int32_t n_codebooks;
    uint32_t seed_lo, seed_hi;
};

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float rbf(float v) { return bf2f(f2bf(v)); }

// 16-byte streaming load of weights: read-only path, do not pollute L1.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Programmatic dependent launch: a kernel launched with the stream-serialization
// attribute may start while its predecessor still runs.  pdl_trigger() lets the
// successor be scheduled; pdl_wait() blocks until the predecessor has finished
// and its writes are visible.  Everything a kernel does before pdl_wait() must
// touch only constants (weights).  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int RT>
__device__ __forceinline__ float pick(const float (&a)[RT], int r) {
    float v = a[0];
#pragma unroll
    for (int i = 1; i < RT; ++i)
        if (r == i) v = a[i];
    return v;
}

// ---------------------------------------------------------------------------
// Embedding gather-sum for a decode step (AudioEmbedding.forward, model.py:559-563)
// plus the per-row (slot, position) table every later kernel of the step reads.
// ---------------------------------------------------------------------------
static __global__ void __launch_bounds__(128) k_embed_codes(
    const int64_t* __restrict__ codes, const int32_t* __restrict__ slots,
    const int32_t* __restrict__ seq_lens, const bf16* __restrict__ table, bf16* __restrict__ x,
    int32_t* __restrict__ row_slot, int32_t* __restrict__ row_pos, int d, int Q, int CS,
    int n_slots, int max_seq, int32_t* __restrict__ flag) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    if (slots) {  // decode step: also publish the row's (slot, position)
        int slot = slots[r];
        if (slot < 0 || slot >= n_slots) {
            if (threadIdx.x == 0) atomicOr(flag, FLAG_BAD_SLOT);
            slot = n_slots - 1;
        }
        if (threadIdx.x == 0) {
            int pos = seq_lens[slot];
            if (pos < 0 || pos >= max_seq) {
                atomicOr(flag, FLAG_BAD_POS);
                pos = pos < 0 ? 0 : max_seq - 1;
            }
            row_slot[r] = slot;
            row_pos[r] = pos;
        }
    }
    // All codes are requested at once, then all table rows, then the rows are added in codebook order (the order the
    // sum is defined in): one dependent round trip instead of one per codebook.
    constexpr int QB = 16;
    for (int k = threadIdx.x * 8; k < d; k += blockDim.x * 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int q0 = 0; q0 < Q; q0 += QB) {
            long long c[QB];
#pragma unroll
            for (int u = 0; u < QB; ++u) c[u] = q0 + u < Q ? codes[(size_t)r * Q + q0 + u] : 0;
            uint4 row[QB];
#pragma unroll
            for (int u = 0; u < QB; ++u) {
                if (c[u] < 0 || c[u] >= CS) {
                    atomicOr(flag, FLAG_BAD_CODE);
                    c[u] = 0;
                }
                row[u] = q0 + u < Q ? __ldg(reinterpret_cast<const uint4*>(table + ((size_t)(q0 + u) * CS + c[u]) * d + k))
                                    : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < QB; ++u) {
                if (q0 + u < Q) {
                    float f[8];
                    unpack8(row[u], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += f[j];
                }
            }
        }
        *reinterpret_cast<uint4*>(x + (size_t)r * d + k) = pack8(acc);
    }
}

// Copies the caller's per-row (slot, position) table of a prefill into the workspace, recording and
// clamping anything outside the cache: every later kernel of the call indexes the KV cache with the
// checked copy, so a bad value can neither read nor write out of bounds.
static __global__ void __launch_bounds__(256) k_check_rows(
    const int32_t* slot_in, const int32_t* pos_in, int32_t* row_slot, int32_t* row_pos, int n, int n_slots,
    int max_seq, int32_t* flag) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int slot = slot_in[i], pos = pos_in[i];
    if (slot < 0 || slot >= n_slots) {
        atomicOr(flag, FLAG_BAD_SLOT);
        slot = slot < 0 ? 0 : n_slots - 1;
    }
    if (pos < 0 || pos >= max_seq) {
        atomicOr(flag, FLAG_BAD_POS);
        pos = pos < 0 ? 0 : max_seq - 1;
    }
    row_slot[i] = slot;
    row_pos[i] = pos;
}

// ---------------------------------------------------------------------------
// Staging functors: fill the CTA's shared activation tile Xs[nr][K] (bf16).
// ---------------------------------------------------------------------------

// RMSNorm (model.py:292-297): fp32 x*rsqrt(mean(x^2)+eps) -> bf16 -> * weight -> bf16.
struct NoPre {};  // nothing to fetch ahead

template <int K>
struct NormW {  // this lane's norm weights
    uint4 w[(K + 255) / 256];
};

struct StageNorm {
    const bf16* x;   // row r of the GEMV lives at x + (r*row_mul + row_add)*K
    const bf16* w;   // (K)
    float eps;
    int row_mul, row_add;
    // single-row form only: the row is x + bf16(sum_p parts[p]), the partial rows (n_parts, K) fp32 that
    // the fused two-kernel layers leave behind (fused_blocks.cuh), added in row order
    const float* parts = nullptr;
    int n_parts = 0;
    // The norm weights are constants: a kernel fetches them before it waits for its predecessor,
    // so that their L2 round trip is not paid between the reduction and the scaling.
    template <int K>
    __device__ __forceinline__ NormW<K> preload() const {
        NormW<K> nw;
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int it = 0; it < (K + 255) / 256; ++it) {
            const int k = it * 256 + lane * 8;
            nw.w[it] = (k < K) ? __ldg(reinterpret_cast<const uint4*>(w + k)) : make_uint4(0, 0, 0, 0);
        }
        return nw;
    }
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr) const {
        stage<K>(Xs, r0, nr, preload<K>());
    }
    // Single row given as x + bf16(sum of partial rows): the whole CTA adds the rows (every thread a few
    // consecutive elements, all rows requested at once, added in row order) and normalises together.
    template <int K>
    __device__ __forceinline__ void stage_parts(bf16* Xs) const {
        constexpr int EPT = K / GEMV_THREADS;  // 2 (K = 512) or 4 (K = 1024)
        static_assert(EPT == 2 || EPT == 4, "partial rows come from the fused layers: K is 512 or 1024");
        constexpr int MAXP = 16;
        __shared__ float red[GEMV_WARPS];
        const int k0 = threadIdx.x * EPT;
        const bf16* xr = x + (size_t)row_add * K;
        float xv[EPT], wv[EPT], sp[EPT];
#pragma unroll
        for (int j = 0; j < EPT; ++j) sp[j] = 0.f;
        if constexpr (EPT == 4) {
            const uint2 xraw = __ldcg(reinterpret_cast<const uint2*>(xr + k0));
            const uint2 wraw = __ldg(reinterpret_cast<const uint2*>(w + k0));
            float4 p[MAXP];
#pragma unroll
            for (int u = 0; u < MAXP; ++u)
                p[u] = u < n_parts ? __ldcg(reinterpret_cast<const float4*>(parts + (size_t)u * K + k0))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < MAXP; ++u) { sp[0] += p[u].x; sp[1] += p[u].y; sp[2] += p[u].z; sp[3] += p[u].w; }
            const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xraw);
            const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wraw);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float2 a = __bfloat1622float2(xh[i]), b = __bfloat1622float2(wh[i]);
                xv[2 * i] = a.x; xv[2 * i + 1] = a.y; wv[2 * i] = b.x; wv[2 * i + 1] = b.y;
            }
        } else {
            const unsigned xraw = __ldcg(reinterpret_cast<const unsigned*>(xr + k0));
            const unsigned wraw = __ldg(reinterpret_cast<const unsigned*>(w + k0));
            float2 p[MAXP];
#pragma unroll
            for (int u = 0; u < MAXP; ++u)
                p[u] = u < n_parts ? __ldcg(reinterpret_cast<const float2*>(parts + (size_t)u * K + k0)) : make_float2(0.f, 0.f);
#pragma unroll
            for (int u = 0; u < MAXP; ++u) { sp[0] += p[u].x; sp[1] += p[u].y; }
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xraw));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wraw));
            xv[0] = a.x; xv[1] = a.y; wv[0] = b.x; wv[1] = b.y;
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            xv[j] = rbf(xv[j] + rbf(sp[j]));
            ss = fmaf(xv[j], xv[j], ss);
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < GEMV_WARPS; ++i) tot += red[i];
        const float rinv = rsqrtf(tot / (float)K + eps);
        if constexpr (EPT == 4) {
            uint2 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
            oh[0] = __floats2bfloat162_rn(rbf(xv[0] * rinv) * wv[0], rbf(xv[1] * rinv) * wv[1]);
            oh[1] = __floats2bfloat162_rn(rbf(xv[2] * rinv) * wv[2], rbf(xv[3] * rinv) * wv[3]);
            *reinterpret_cast<uint2*>(Xs + k0) = o;
        } else {
            *reinterpret_cast<__nv_bfloat162*>(Xs + k0) =
                __floats2bfloat162_rn(rbf(xv[0] * rinv) * wv[0], rbf(xv[1] * rinv) * wv[1]);
        }
    }
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr, const NormW<K>& nw) const {
        if constexpr (K == 512 || K == 1024) {
            if (n_parts > 0) {  // uniform over the CTA
                stage_parts<K>(Xs);
                return;
            }
        }
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int rr = warp; rr < nr; rr += (int)(blockDim.x >> 5)) {
            const bf16* xr = x + ((size_t)(r0 + rr) * row_mul + row_add) * K;
            constexpr int IT = (K + 255) / 256;
            float v[IT][8];
            float ss = 0.f;
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int k = it * 256 + lane * 8;
                if (k < K) {
                    uint4 u = __ldcg(reinterpret_cast<const uint4*>(xr + k));
                    unpack8(u, v[it]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss = fmaf(v[it][j], v[it][j], ss);
                }
            }
            ss = warp_sum(ss);
            const float rinv = rsqrtf(ss / (float)K + eps);
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int k = it * 256 + lane * 8;
                if (k < K) {
                    float wf[8], o[8];
                    unpack8(nw.w[it], wf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = rbf(v[it][j] * rinv) * wf[j];
                    *reinterpret_cast<uint4*>(Xs + rr * K + k) = pack8(o);
                }
            }
        }
    }
};

struct StageCopy {
    const bf16* x;  // (M, K)
    template <int K>
    __device__ __forceinline__ NoPre preload() const { return NoPre{}; }
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr, const NoPre&) const { stage<K>(Xs, r0, nr); }
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr) const {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)r0 * K);
        uint4* dst = reinterpret_cast<uint4*>(Xs);
        for (int i = threadIdx.x; i < nr * (K / 8); i += blockDim.x) dst[i] = __ldcg(src + i);
    }
};

// Online-softmax state merge helpers (fp32, finite sentinel instead of -inf).
constexpr float NEG_BIG = -1.0e30f;

// Depth-transformer attention (RQBlock.forward_kv, model.py:613-635; SDPA math
// backend: fp32 softmax over <= Q keys, scale 1/8) computed straight into the
// tile that feeds out_proj.  One warp per head; lane = (key group g, 8-dim chunk s).
struct StageRqAttn {
    const bf16* q;    // (M, H*64)
    const bf16* kc;   // (R, Qpos, H*64) this layer
    const bf16* vc;
    int H;            // heads
    int Qpos;         // positions per row in the cache (n_quantizers)
    int rows_per_b;   // row r -> b = r / rows_per_b, pos = pos_base + r % rows_per_b
    int pos_base;
    template <int K>
    __device__ __forceinline__ NoPre preload() const { return NoPre{}; }
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr, const NoPre&) const { stage<K>(Xs, r0, nr); }
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr) const {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int s = lane & 7, g = lane >> 3;
        for (int rr = 0; rr < nr; ++rr) {
            const int r = r0 + rr;
            const int b = r / rows_per_b, pos = pos_base + r % rows_per_b;
            for (int h = warp; h < H; h += (int)(blockDim.x >> 5)) {
                // q and every key/value group of this lane (<= 16 positions = 4 groups) are requested
                // together: one L2 round trip instead of one per group of four positions
                const uint4 qraw = __ldcg(reinterpret_cast<const uint4*>(q + (size_t)r * K + h * HD + s * 8));
                uint4 kraw[4], vraw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int t = u * 4 + g;
                    const bool ok = t <= pos;
                    const size_t off = ((size_t)b * Qpos + (ok ? t : 0)) * K + h * HD + s * 8;
                    if (u * 4 <= pos) {
                        kraw[u] = __ldcg(reinterpret_cast<const uint4*>(kc + off));
                        vraw[u] = __ldcg(reinterpret_cast<const uint4*>(vc + off));
                    } else {
                        kraw[u] = make_uint4(0, 0, 0, 0);
                        vraw[u] = make_uint4(0, 0, 0, 0);
                    }
                }
                float qf[8];
                unpack8(qraw, qf);
                float m = NEG_BIG, l = 0.f, acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (u * 4 <= pos) {  // the whole warp runs the same groups
                        const int t = u * 4 + g;
                        const bool ok = t <= pos;
                        float kf[8], vf[8];
                        unpack8(kraw[u], kf);
                        unpack8(vraw[u], vf);
                        float d = 0.f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) d = fmaf(qf[j], kf[j], d);
                        d += __shfl_xor_sync(0xffffffffu, d, 1);
                        d += __shfl_xor_sync(0xffffffffu, d, 2);
                        d += __shfl_xor_sync(0xffffffffu, d, 4);
                        if (ok) {
                            const float sc = d * 0.125f;
                            const float mn = fmaxf(m, sc);
                            const float corr = __expf(m - mn), p = __expf(sc - mn);
                            l = l * corr + p;
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc[j] = fmaf(p, vf[j], acc[j] * corr);
                            m = mn;
                        }
                    }
                }
#pragma unroll
                for (int o = 8; o <= 16; o <<= 1) {
                    const float mo = __shfl_xor_sync(0xffffffffu, m, o);
                    const float lo = __shfl_xor_sync(0xffffffffu, l, o);
                    const float mn = fmaxf(m, mo);
                    const float ca = __expf(m - mn), cb = __expf(mo - mn);
                    l = l * ca + lo * cb;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float ao = __shfl_xor_sync(0xffffffffu, acc[j], o);
                        acc[j] = acc[j] * ca + ao * cb;
                    }
                    m = mn;
                }
                if (g == 0) {
                    const float inv = 1.f / l;
                    float o8[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o8[j] = acc[j] * inv;
                    *reinterpret_cast<uint4*>(Xs + rr * K + h * HD + s * 8) = pack8(o8);
                }
            }
        }
    }
};

// ---------------------------------------------------------------------------
// Epilogue functors: which weight rows a work item reads, and what to do with
// the RT sums per weight row.  After the butterfly reduction every lane holds all
// sums; lane r finishes activation row r.
// ---------------------------------------------------------------------------

// Wqkv (+ RoPE on q,k) with K/V written straight into the cache (MHA.forward_flash,
// model.py:220-257; rope.py:16-57).  Work item = one interleaved pair (2i, 2i+1).
struct EpiQkv {
    const bf16* W;      // (N, K)
    int K;
    bf16* q_out;        // (M, q_cols)
    int q_cols, kv_cols;
    bf16* k_cache;      // this layer
    bf16* v_cache;
    const int32_t* row_slot;  // NULL -> depth-transformer addressing below
    const int32_t* row_pos;
    int max_seq;              // positions per slot in the cache
    const bf16* rope;         // (max_seq, 64, 2) or NULL
    int rows_per_b, pos_base; // used when row_slot == NULL
    int kv_hint;              // 1: prefetch the K/V rows of the attention that follows into L2
    static constexpr int NC = 2;
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[2]) const {
        wr[0] = W + (size_t)(2 * item) * K;
        wr[1] = wr[0] + K;
    }
    // Warm L2 (and the TLB) with the K/V rows the attention kernel that follows will read: the
    // rows before each stream's current position do not change during the frame.  The whole
    // grid shares the work, one 128-byte line per thread and step.  Two steps, so that the
    // round trip for (slot, position) is not paid in front of the staging loads: lane r asks
    // for row r's pair first thing, the prefetches are issued once the tile is staged.
    struct Hint {
        int slot, pos;
    };
    __device__ __forceinline__ Hint hint_begin(int M) const {
        Hint h{0, 0};
        const int lane = threadIdx.x & 31;
        if (row_slot && kv_hint && lane < M) {
            h.slot = __ldcg(row_slot + lane);
            h.pos = __ldcg(row_pos + lane);
        }
        return h;
    }
    __device__ __forceinline__ void hint_end(int M, const Hint& h) const {
        if (!row_slot || !kv_hint) return;
        const size_t row_bytes = (size_t)kv_cols * sizeof(bf16);
        const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
        for (int r = 0; r < M && r < 32; ++r) {
            const int slot = __shfl_sync(0xffffffffu, h.slot, r), pos = __shfl_sync(0xffffffffu, h.pos, r);
            const size_t lines = (size_t)pos * row_bytes / 128;
            const char* kb = reinterpret_cast<const char*>(k_cache) + (size_t)slot * max_seq * row_bytes;
            const char* vb = reinterpret_cast<const char*>(v_cache) + (size_t)slot * max_seq * row_bytes;
            for (size_t i = tid; i < 2 * lines; i += nth) {
                const char* p = i < lines ? kb + i * 128 : vb + (i - lines) * 128;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
            }
        }
    }
    // What lane r needs for row r besides the sums: requested before the dot products, so that the
    // two dependent L2 round trips (position, then RoPE factors) are not paid after them.
    struct Pre {
        int slot, pos;
        float c0, s0, c1, s1;
    };
    __device__ __forceinline__ Pre pre(int item, int r0, int nr, int lane) const {
        Pre p{0, 0, 1.f, 0.f, 1.f, 0.f};
        if (lane >= nr) return p;
        const int r = r0 + lane;
        const int n = 2 * item;
        if (row_slot) {
            p.slot = __ldcg(row_slot + r);
            p.pos = __ldcg(row_pos + r);
        } else {
            p.slot = r / rows_per_b;
            p.pos = pos_base + r % rows_per_b;
        }
        if (rope && n < q_cols + kv_cols) {
            const int dd = n & (HD - 1);
            const uint2 f = __ldg(reinterpret_cast<const uint2*>(rope + ((size_t)p.pos * HD + dd) * 2));
            p.c0 = bf2f(__ushort_as_bfloat16((unsigned short)(f.x & 0xffffu)));
            p.s0 = bf2f(__ushort_as_bfloat16((unsigned short)(f.x >> 16)));
            p.c1 = bf2f(__ushort_as_bfloat16((unsigned short)(f.y & 0xffffu)));
            p.s1 = bf2f(__ushort_as_bfloat16((unsigned short)(f.y >> 16)));
        }
        return p;
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[2][RT]) const {
        store<RT>(item, r0, nr, lane, acc, pre(item, r0, nr, lane));
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[2][RT], const Pre& pr_) const {
        if (lane >= nr) return;
        const int r = r0 + lane;
        const int n = 2 * item;
        float t0 = rbf(pick<RT>(acc[0], lane)), t1 = rbf(pick<RT>(acc[1], lane));
        const int slot = pr_.slot, pos = pr_.pos;
        if (rope && n < q_cols + kv_cols) {
            const float c0 = pr_.c0, s0 = pr_.s0, c1 = pr_.c1, s1 = pr_.s1;
            // t*cos + rotate_half(t)*sin, each product and the sum rounded to bf16
            const float o0 = rbf(rbf(t0 * c0) + rbf((-t1) * s0));
            const float o1 = rbf(rbf(t1 * c1) + rbf(t0 * s1));
            t0 = o0;
            t1 = o1;
        }
        __nv_bfloat162 pr = __floats2bfloat162_rn(t0, t1);
        if (n < q_cols) {
            *reinterpret_cast<__nv_bfloat162*>(q_out + (size_t)r * q_cols + n) = pr;
        } else if (n < q_cols + kv_cols) {
            *reinterpret_cast<__nv_bfloat162*>(
                k_cache + ((size_t)slot * max_seq + pos) * kv_cols + (n - q_cols)) = pr;
        } else {
            *reinterpret_cast<__nv_bfloat162*>(
                v_cache + ((size_t)slot * max_seq + pos) * kv_cols + (n - q_cols - kv_cols)) = pr;
        }
    }
};

// x += bf16(W a): out_proj and w2 with the residual add (model.py:367, 374).
struct EpiResidual {
    const bf16* W;  // (N, K)
    int K;
    bf16* x;        // (M, N) residual stream, updated in place
    int N;
    bf16* tap;      // optional copy of the new x (M, N)
    static constexpr int NC = 1;
    typedef NoPre Hint;
    __device__ __forceinline__ Hint hint_begin(int) const { return NoPre{}; }
    __device__ __forceinline__ void hint_end(int, const NoPre&) const {}
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[1]) const {
        wr[0] = W + (size_t)item * K;
    }
    // The element this lane adds to: requested before the dot products hide its L2 round trip.
    typedef unsigned short Pre;
    __device__ __forceinline__ Pre pre(int item, int r0, int nr, int lane) const {
        if (lane >= nr) return 0;
        return __ldcg(reinterpret_cast<const unsigned short*>(x) + (size_t)(r0 + lane) * N + item);
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[1][RT]) const {
        store<RT>(item, r0, nr, lane, acc, pre(item, r0, nr, lane));
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[1][RT], Pre xb) const {
        if (lane >= nr) return;
        const size_t idx = (size_t)(r0 + lane) * N + item;
        const bf16 o = f2bf(bf2f(__ushort_as_bfloat16(xb)) + rbf(pick<RT>(acc[0], lane)));
        x[idx] = o;
        if (tap) tap[idx] = o;
    }
};

// silu(w1 h) * (w3 h)  (LlamaMLP.forward, model.py:282-283); item = hidden unit n.
struct EpiSwiGLU {
    const bf16* W1;
    const bf16* W3;
    int K;
    bf16* act;  // (M, F)
    int F;
    static constexpr int NC = 2;
    typedef NoPre Hint;
    __device__ __forceinline__ Hint hint_begin(int) const { return NoPre{}; }
    __device__ __forceinline__ void hint_end(int, const NoPre&) const {}
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[2]) const {
        wr[0] = W1 + (size_t)item * K;
        wr[1] = W3 + (size_t)item * K;
    }
    typedef NoPre Pre;
    __device__ __forceinline__ Pre pre(int, int, int, int) const { return NoPre{}; }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[2][RT], const NoPre&) const {
        store<RT>(item, r0, nr, lane, acc);
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[2][RT]) const {
        if (lane >= nr) return;
        const float a = rbf(pick<RT>(acc[0], lane)), g = rbf(pick<RT>(acc[1], lane));
        const float s = rbf(a / (1.0f + expf(-a)));
        act[(size_t)(r0 + lane) * F + item] = f2bf(s * g);
    }
};

// Plain bf16 output rows: codec_head / eos_head (item == n_main -> extra row with
// bias, model.py:1099) and the depth-transformer heads.
struct EpiLogits {
    const bf16* W;      // (n_main, K)
    int K;
    int n_main;
    bf16* out;          // (M, n_main)
    const bf16* W_extra;  // (1, K) or NULL
    const bf16* b_extra;  // (1)
    bf16* out_extra;      // (M)
    bf16* tap;            // optional second copy of out with its own row stride
    int tap_stride;
    static constexpr int NC = 1;
    typedef NoPre Hint;
    __device__ __forceinline__ Hint hint_begin(int) const { return NoPre{}; }
    __device__ __forceinline__ void hint_end(int, const NoPre&) const {}
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[1]) const {
        wr[0] = item < n_main ? W + (size_t)item * K : W_extra;
    }
    typedef NoPre Pre;
    __device__ __forceinline__ Pre pre(int, int, int, int) const { return NoPre{}; }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[1][RT], const NoPre&) const {
        store<RT>(item, r0, nr, lane, acc);
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[1][RT]) const {
        if (lane >= nr) return;
        const int r = r0 + lane;
        const float v = pick<RT>(acc[0], lane);
        if (item < n_main) {
            const bf16 o = f2bf(v);
            out[(size_t)r * n_main + item] = o;
            if (tap) tap[(size_t)r * tap_stride + item] = o;
        } else {
            out_extra[r] = f2bf(v + bf2f(b_extra[0]));
        }
    }
};

// Depth-transformer position 0: backbone_proj(hidden) + pos_emb[0] (model.py:921).
struct EpiProjPos {
    const bf16* W;    // (rd, K)
    int K;
    const bf16* pos_emb;  // row 0
    bf16* out;        // (rows_out, rd); row of stream b is b*row_mul
    int rd, row_mul;
    static constexpr int NC = 1;
    typedef NoPre Hint;
    __device__ __forceinline__ Hint hint_begin(int) const { return NoPre{}; }
    __device__ __forceinline__ void hint_end(int, const NoPre&) const {}
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[1]) const {
        wr[0] = W + (size_t)item * K;
    }
    typedef NoPre Pre;
    __device__ __forceinline__ Pre pre(int, int, int, int) const { return NoPre{}; }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[1][RT], const NoPre&) const {
        store<RT>(item, r0, nr, lane, acc);
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane,
                                          const float (&acc)[1][RT]) const {
        if (lane >= nr) return;
        const int b = r0 + lane;
        out[(size_t)b * row_mul * rd + item] =
            f2bf(rbf(pick<RT>(acc[0], lane)) + bf2f(pos_emb[item]));
    }
};

// ---------------------------------------------------------------------------
// The batched GEMV.  Each warp keeps its 1-2 weight rows in registers (loaded
// once, 16 bytes per lane per request, all requests in flight before any use)
// and sweeps the M activation rows in tiles of RT staged in shared memory.
// ---------------------------------------------------------------------------
template <int K, int RT, class Stage, class Epi>
__global__ void __launch_bounds__(GEMV_THREADS, (RT >= 4 ? 2 : 1)) k_gemv(Stage st, Epi ep, int M, int n_items) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Xs = reinterpret_cast<bf16*>(smem_raw);
    constexpr int NC = Epi::NC;
    constexpr int IT = (K + 255) / 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * GEMV_WARPS + warp;
    const bool live = item < n_items;
    pdl_trigger();

    uint4 w[NC][IT];
    if (live) {
        const bf16* wr[NC];
        ep.rows(item, wr);
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int k = it * 256 + lane * 8;
                w[c][it] = (k < K) ? ldg_stream(wr[c] + k) : make_uint4(0, 0, 0, 0);
            }
    }
    const auto nw = st.template preload<K>();  // constants too
    pdl_wait();  // the weights above are constants; activations below come from the predecessor
    const typename Epi::Hint hint = ep.hint_begin(M);
    for (int r0 = 0; r0 < M; r0 += RT) {
        const int nr = min(RT, M - r0);
        // what the epilogue needs from global memory is requested now and used after the dot products
        typename Epi::Pre pre = live ? ep.pre(item, r0, nr, lane) : typename Epi::Pre{};
        if (r0) __syncthreads();
        st.template stage<K>(Xs, r0, nr, nw);
        __syncthreads();
        if (r0 == 0) ep.hint_end(M, hint);  // its (slot, position) pair arrived while the tile was staged
        if (live) {
            float acc[NC][RT];
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int r = 0; r < RT; ++r) acc[c][r] = 0.f;
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int k = it * 256 + lane * 8;
                if (k < K) {
                    float wf[NC][8];
#pragma unroll
                    for (int c = 0; c < NC; ++c) unpack8(w[c][it], wf[c]);
#pragma unroll
                    for (int r = 0; r < RT; ++r) {
                        if (r < nr) {
                            float xf[8];
                            unpack8(*reinterpret_cast<const uint4*>(Xs + r * K + k), xf);
#pragma unroll
                            for (int c = 0; c < NC; ++c)
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    acc[c][r] = fmaf(wf[c][j], xf[j], acc[c][r]);
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int r = 0; r < RT; ++r) acc[c][r] = warp_sum(acc[c][r]);
            ep.template store<RT>(item, r0, nr, lane, acc, pre);
        }
    }
}

// ---------------------------------------------------------------------------
// Backbone decode attention (flash_attn_with_kvcache call, model.py:247-257):
// ragged per-row length row_pos[r]+1, GQA 2:1, scale 1/8, fp32 softmax.  One CTA
// = (split of ATT_SPLIT keys, kv head, row); partial (acc, m, l) per split go to
// scratch and the last CTA of a (row, kv head) merges them in split order, so the
// result does not depend on arrival order.
// ---------------------------------------------------------------------------
struct AttnArgs {
    const bf16* q;        // (R, Hq*64)
    const bf16* kc;       // (slots, max_seq, Hkv, 64) this layer
    const bf16* vc;
    const int32_t* row_slot;
    const int32_t* row_pos;
    float* part;          // (R, Hq, S, PART_STRIDE)
    int32_t* counters;    // (R, Hkv), zero between launches
    bf16* out;            // (R, Hq*64)
    int Hq, Hkv, max_seq, S;
    unsigned long long* dbg;  // optional: 8 device-clock stamps of one unit (profiling aid)
    int n_slots;              // slots in the cache; 0 = unknown (only negative slots can then be caught)
    int32_t* flag;            // device error word (may be NULL)
};

__device__ __forceinline__ void attn_stamp(const AttnArgs& a, int tid, int i) {
    if (a.dbg && tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.dbg[i] = t;
    }
}

__device__ __forceinline__ void softmax_merge(float& m, float& l, float (&acc)[8], float mo,
                                              float lo, const float (&ao)[8]) {
    const float mn = fmaxf(m, mo);
    const float ca = __expf(m - mn), cb = __expf(mo - mn);
    l = l * ca + lo * cb;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = acc[j] * ca + ao[j] * cb;
    m = mn;
}

// Named barrier over `n` threads (id 0 with n = blockDim.x is __syncthreads()).
__device__ __forceinline__ void bar_named(int id, int n) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}

struct AttnSmem {
    float sm[4][2][8][10];  // [warp][head][s][acc8, m, l]
    int s_last;
};

// One (split, kv head, row) unit of work for a group of ATT_THREADS threads whose
// index within the group is `tid`; the group synchronises on named barrier bar_id.
__device__ __forceinline__ void attn_unit(const AttnArgs& a, int sp, int kvh, int r, int tid,
                                          AttnSmem& S_, int bar_id) {
    attn_stamp(a, tid, 0);
    int slot = __ldcg(a.row_slot + r);  // both requests in flight before the first use
    int pos = __ldcg(a.row_pos + r);
    // A slot or position outside the cache is recorded and clamped, never followed: a position past
    // max_seq would also ask for more splits than the grid has, and the merge would never run.
    if (slot < 0 || (a.n_slots > 0 && slot >= a.n_slots)) {
        if (a.flag && tid == 0 && sp == 0 && kvh == 0) atomicOr(a.flag, FLAG_BAD_SLOT);
        slot = slot < 0 ? 0 : a.n_slots - 1;
    }
    if (pos < 0 || pos >= a.max_seq) {
        if (a.flag && tid == 0 && sp == 0 && kvh == 0) atomicOr(a.flag, FLAG_BAD_POS);
        pos = pos < 0 ? 0 : a.max_seq - 1;
    }
    const int len = pos + 1;
    const int nsplit = (len + ATT_SPLIT - 1) / ATT_SPLIT;
    if (sp >= nsplit) return;
    const int warp = tid >> 5, lane = tid & 31;
    const int s = lane & 7, g = lane >> 3;
    const int G = a.Hq / a.Hkv;  // q heads per kv head (2)
    const int t_begin = sp * ATT_SPLIT, t_end = min(len, t_begin + ATT_SPLIT);
    const size_t pos_stride = (size_t)a.Hkv * HD;
    const bf16* kb = a.kc + (size_t)slot * a.max_seq * pos_stride + kvh * HD + s * 8;
    const bf16* vb = a.vc + (size_t)slot * a.max_seq * pos_stride + kvh * HD + s * 8;

    // all K and V requests of this lane in flight before any arithmetic
    uint4 kr[ATT_ITERS], vr[ATT_ITERS];
#pragma unroll
    for (int it = 0; it < ATT_ITERS; ++it) {
        const int t = t_begin + it * 16 + warp * 4 + g;
        if (t < t_end) {
            kr[it] = ldg_stream(kb + (size_t)t * pos_stride);
            vr[it] = ldg_stream(vb + (size_t)t * pos_stride);
        } else {
            kr[it] = make_uint4(0, 0, 0, 0);
            vr[it] = make_uint4(0, 0, 0, 0);
        }
    }
    float (&sm)[4][2][8][10] = S_.sm;
    int& s_last = S_.s_last;
    float qf[2][8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int hq = kvh * G + (h < G ? h : 0);
        unpack8(__ldcg(reinterpret_cast<const uint4*>(a.q + (size_t)r * a.Hq * HD + hq * HD + s * 8)), qf[h]);
    }
    attn_stamp(a, tid, 1);
    float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f}, acc[2][8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[h][j] = 0.f;

#pragma unroll
    for (int it = 0; it < ATT_ITERS; ++it) {
        const int t = t_begin + it * 16 + warp * 4 + g;
        float kf[8], vf[8];
        unpack8(kr[it], kf);
        unpack8(vr[it], vf);
        float d[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float dd = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) dd = fmaf(qf[h][j], kf[j], dd);
            dd += __shfl_xor_sync(0xffffffffu, dd, 1);
            dd += __shfl_xor_sync(0xffffffffu, dd, 2);
            dd += __shfl_xor_sync(0xffffffffu, dd, 4);
            d[h] = dd * 0.125f;
        }
        if (t < t_end) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mn = fmaxf(m[h], d[h]);
                const float corr = __expf(m[h] - mn), p = __expf(d[h] - mn);
                l[h] = l[h] * corr + p;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[h][j] = fmaf(p, vf[j], acc[h][j] * corr);
                m[h] = mn;
            }
        }
    }
    attn_stamp(a, tid, 2);
    // merge the 4 key groups of the warp
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[h], o);
            const float lo = __shfl_xor_sync(0xffffffffu, l[h], o);
            float ao[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) ao[j] = __shfl_xor_sync(0xffffffffu, acc[h][j], o);
            softmax_merge(m[h], l[h], acc[h], mo, lo, ao);
        }
    }
    if (g == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 8; ++j) sm[warp][h][s][j] = acc[h][j];
            sm[warp][h][s][8] = m[h];
            sm[warp][h][s][9] = l[h];
        }
    }
    attn_stamp(a, tid, 3);
    bar_named(bar_id, ATT_THREADS);
    // thread (h, dim): merge the 4 warps
    const int h = tid >> 6, dim = tid & 63;
    const int ds = dim >> 3, dj = dim & 7;
    float M_ = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; ++w) M_ = fmaxf(M_, sm[w][h][ds][8]);
    float L_ = 0.f, O_ = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float c = __expf(sm[w][h][ds][8] - M_);
        L_ += sm[w][h][ds][9] * c;
        O_ += sm[w][h][ds][dj] * c;
    }
    const bool head_ok = h < G;
    const int hq = kvh * G + (head_ok ? h : 0);
    if (nsplit == 1) {
        if (head_ok) a.out[(size_t)r * a.Hq * HD + hq * HD + dim] = f2bf(O_ / L_);
        return;
    }
    float* pp = a.part + (((size_t)r * a.Hq + hq) * a.S + sp) * PART_STRIDE;
    if (head_ok) {
        pp[dim] = O_;
        if (dim == 0) {
            pp[HD] = M_;
            pp[HD + 1] = L_;
        }
    }
    attn_stamp(a, tid, 4);
    bar_named(bar_id, ATT_THREADS);  // every thread's partial stores precede thread 0's release below
    attn_stamp(a, tid, 5);
    if (tid == 0) {
        int old;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(a.counters + r * a.Hkv + kvh) : "memory");
        s_last = (old == nsplit - 1);
    }
    bar_named(bar_id, ATT_THREADS);
    attn_stamp(a, tid, 6);
    if (!s_last) return;
    if (head_ok) {
        // merge the splits in index order; 16 splits' worth of loads are in flight at a time
        const float* pb = a.part + ((size_t)r * a.Hq + hq) * a.S * PART_STRIDE;
        float Mx = NEG_BIG, Ls = 0.f, Os = 0.f;
        for (int i0 = 0; i0 < nsplit; i0 += 16) {
            float ms[16], ls[16], os[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const bool ok = i0 + u < nsplit;
                const float* q = pb + (size_t)(ok ? i0 + u : i0) * PART_STRIDE;
                ms[u] = ok ? __ldcg(q + HD) : NEG_BIG;
                ls[u] = ok ? __ldcg(q + HD + 1) : 0.f;
                os[u] = ok ? __ldcg(q + dim) : 0.f;
            }
            float Mn = Mx;
#pragma unroll
            for (int u = 0; u < 16; ++u) Mn = fmaxf(Mn, ms[u]);
            const float c0 = __expf(Mx - Mn);
            Ls *= c0;
            Os *= c0;
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const float c = __expf(ms[u] - Mn);
                Ls += ls[u] * c;
                Os += os[u] * c;
            }
            Mx = Mn;
        }
        a.out[(size_t)r * a.Hq * HD + hq * HD + dim] = f2bf(Os / Ls);
    }
    if (tid == 0) a.counters[r * a.Hkv + kvh] = 0;
}

static __global__ void __launch_bounds__(ATT_THREADS) k_attn_decode(AttnArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ AttnSmem S_;
    attn_unit(a, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x, S_, 0);
}

// ---------------------------------------------------------------------------
// Final RMSNorm of the backbone -> hidden_out, and seq_lens[slot] += inc.
// (Decoder.forward_flash model.py:548-549; engine.py:449, 502.)
// ---------------------------------------------------------------------------
static __global__ void __launch_bounds__(128) k_final_norm(const bf16* __restrict__ x,
                                                    const bf16* __restrict__ w, float eps,
                                                    bf16* __restrict__ out, int d,
                                                    const int32_t* __restrict__ row_slot,
                                                    const int32_t* __restrict__ seq_inc,
                                                    int32_t* __restrict__ seq_lens, int bump,
                                                    const float* __restrict__ parts, int n_parts,
                                                    bf16* __restrict__ xsum_out) {
    pdl_trigger();
    // the norm weights do not depend on the previous kernel (single pass over d <= 1024: one piece per thread)
    float wf0[8];
    {
        const int k = threadIdx.x * 8;
        unpack8(k < d ? __ldg(reinterpret_cast<const uint4*>(w + k)) : make_uint4(0, 0, 0, 0), wf0);
    }
    pdl_wait();
    const int r = blockIdx.x;
    __shared__ float red[4];
    __shared__ __align__(16) bf16 xsum[1024];
    const bf16* xr = x + (size_t)r * d;
    if (n_parts > 0) {
        // single row, d <= 1024: x + bf16(sum of the fused layers' partial rows), kept for the second pass
        for (int k = threadIdx.x * 8; k < d; k += 128 * 8) {
            float f[8], sp[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            unpack8(__ldcg(reinterpret_cast<const uint4*>(xr + k)), f);
            for (int p0 = 0; p0 < n_parts; p0 += 16) {  // sixteen rows in flight at a time, added in row order
                float4 pa[16], pb[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const bool ok = p0 + u < n_parts;
                    const float* q = parts + (size_t)(ok ? p0 + u : p0) * d + k;
                    pa[u] = ok ? __ldcg(reinterpret_cast<const float4*>(q)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    pb[u] = ok ? __ldcg(reinterpret_cast<const float4*>(q + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    sp[0] += pa[u].x; sp[1] += pa[u].y; sp[2] += pa[u].z; sp[3] += pa[u].w;
                    sp[4] += pb[u].x; sp[5] += pb[u].y; sp[6] += pb[u].z; sp[7] += pb[u].w;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = rbf(f[j] + rbf(sp[j]));
            const uint4 u = pack8(f);
            *reinterpret_cast<uint4*>(xsum + k) = u;
            if (xsum_out) *reinterpret_cast<uint4*>(xsum_out + k) = u;
        }
        __syncthreads();
        xr = xsum;
    }
    float ss = 0.f;
    for (int k = threadIdx.x * 8; k < d; k += 128 * 8) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + k), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float tot = red[0] + red[1] + red[2] + red[3];
    const float rinv = rsqrtf(tot / (float)d + eps);
    for (int k = threadIdx.x * 8; k < d; k += 128 * 8) {
        float f[8], wf[8], o[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + k), f);
        if (k == (int)threadIdx.x * 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) wf[j] = wf0[j];
        } else {
            unpack8(__ldg(reinterpret_cast<const uint4*>(w + k)), wf);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rbf(f[j] * rinv) * wf[j];
        *reinterpret_cast<uint4*>(out + (size_t)r * d + k) = pack8(o);
    }
    if (bump && threadIdx.x == 0) {
        const int inc = seq_inc ? seq_inc[r] : 1;
        if (inc) seq_lens[row_slot[r]] += inc;
    }
}

// ---------------------------------------------------------------------------
// Sampler: one CTA per row over CS = 2048 logits.
//   cb0 (engine.py:571-590, 855-863): optional repetition penalty, then greedy or
//       softmax(l/T) restricted to the top-k, inverse-CDF draw.
//   depth codebooks (model.py:955-962): l/T, keep entries >= k-th value, softmax,
//       draw.  Greedy = first index of the maximum (torch.argmax).
// Uniforms come from Philox4x32-10 keyed (seed; slot, frame counter, codebook).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct SampleArgs {
    const bf16* logits;       // (B, CS) rows with stride `stride`
    int stride;
    const SamplingCtl* ctl;
    const int32_t* slots;     // (B)
    int32_t* frame_ctr;       // (n_slots)
    int codebook;             // 0 = cb0
    int first_frame;          // cb0 of a chunk's first frame: no top-k
    float* rep_counts;        // (n_slots, CS) cb0 only
    int32_t* rep_hist;        // (n_slots, REP_HIST_MAX)
    int32_t* rep_head;        // (n_slots)
    int32_t* rep_filled;      // (n_slots)
    int32_t* code_cur;        // (B) out
    int64_t* codes_out;       // (B, Q) out, column out_col
    int Q, out_col;
    const bf16* eos_logit;    // (B) optional, cb0 only
    float* eos_prob;          // (B)
    int bump_frame;           // last sampler of the frame advances frame_ctr
    int zero_from;            // >0: also zero codes_out[r, zero_from..Q)
    // optional: also build the depth token the next codebook consumes,
    // emb_out[r*emb_row_mul + emb_row_add] = code_emb[(emb_p-1)*CS + code] + pos_emb[emb_p]
    // (model.py:922-925, 967-969)
    bf16* emb_out;
    const bf16* code_emb;
    const bf16* pos_emb;
    int emb_p, emb_rd, emb_row_mul, emb_row_add;
    // optional, cb0 only: stats_out[2r] = entropy (nats) and stats_out[2r+1] = largest probability of
    // softmax(penalised logits / temperature) over the whole codebook - what the reference's streaming
    // gate averages over the first frames of a chunk (engine.py:1369-1372, 1418-1424, 1455-1460)
    float* stats_out;
    int n_slots;              // per-slot state has this many entries: a slot outside is recorded and clamped
    int32_t* flag;
};

struct SampleSmem {
    float s_f[8];
    int s_i[8];
    uint32_t hist[256];
    uint32_t s_prefix, s_krem;
    int s_pick, s_lastkept;
};

// Samples row r with a group of SAMPLE_THREADS threads (index `tid` in the group,
// named barrier bar_id).  Returns the chosen code to every thread of the group.
__device__ __forceinline__ int sample_row(const SampleArgs& a, int r, int tid, SampleSmem& S_, int bar_id) {
    constexpr int CS = SAMPLE_THREADS * SAMPLE_EL;
    const int warp = tid >> 5, lane = tid & 31;
    // the row's logits are requested before anything waits for the slot (one dependent round trip less)
    const uint4 raw_logits = __ldcg(reinterpret_cast<const uint4*>(a.logits + (size_t)r * a.stride + tid * SAMPLE_EL));
    int slot = __ldcg(a.slots + r);
    if (slot < 0 || slot >= a.n_slots) {
        if (a.flag && tid == 0) atomicOr(a.flag, FLAG_BAD_SLOT);
        slot = slot < 0 ? 0 : a.n_slots - 1;
    }
    const SamplingCtl ctl = *a.ctl;
    const bool is_cb0 = a.codebook == 0;
    float (&s_f)[8] = S_.s_f;
    int (&s_i)[8] = S_.s_i;
    uint32_t (&hist)[256] = S_.hist;
    uint32_t& s_prefix = S_.s_prefix;
    uint32_t& s_krem = S_.s_krem;
    int& s_pick = S_.s_pick;
    int& s_lastkept = S_.s_lastkept;

    const uint32_t frame_no = (uint32_t)a.frame_ctr[slot];   // for the draw's Philox key, asked for early
    float v[SAMPLE_EL];
    unpack8(raw_logits, v);
    if (is_cb0 && ctl.rep_penalty > 1.0f) {
        const float* cnt = a.rep_counts + (size_t)slot * CS + tid * SAMPLE_EL;
#pragma unroll
        for (int j = 0; j < SAMPLE_EL; ++j) {
            const float c = cnt[j];
            if (c != 0.f) {
                const float f = powf(ctl.rep_penalty, c);
                v[j] = v[j] > 0.f ? v[j] / f : v[j] * f;
            }
        }
    }
    int top_k = is_cb0 ? (a.first_frame && ctl.top_k_cb0 != 1 ? 0 : ctl.top_k_cb0) : ctl.top_k_rq;
    if (top_k >= CS) top_k = 0;

    // block argmax, first index on ties
    float bv = v[0];
    int bi = tid * SAMPLE_EL;
#pragma unroll
    for (int j = 1; j < SAMPLE_EL; ++j)
        if (v[j] > bv) { bv = v[j]; bi = tid * SAMPLE_EL + j; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { s_f[warp] = bv; s_i[warp] = bi; }
    bar_named(bar_id, SAMPLE_THREADS);
    bv = s_f[0]; bi = s_i[0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
        if (s_f[w] > bv || (s_f[w] == bv && s_i[w] < bi)) { bv = s_f[w]; bi = s_i[w]; }
    bar_named(bar_id, SAMPLE_THREADS);

    if (is_cb0 && a.stats_out) {
        // H = log Z - sum e_i x_i / Z with x_i = (v_i - max) / T, e_i = exp(x_i); p_max = 1 / Z
        const float invT = 1.0f / ctl.temperature;
        float z = 0.f, sx = 0.f;
#pragma unroll
        for (int j = 0; j < SAMPLE_EL; ++j) {
            const float x = (v[j] - bv) * invT;
            const float e = expf(x);
            z += e;
            sx = fmaf(e, x, sx);
        }
        z = warp_sum(z);
        sx = warp_sum(sx);
        float* scr = reinterpret_cast<float*>(hist);  // free until the k-th value search clears it
        if (lane == 0) { scr[warp] = z; scr[8 + warp] = sx; }
        bar_named(bar_id, SAMPLE_THREADS);
        if (tid == 0) {
            float Z = 0.f, SX = 0.f;
            for (int w = 0; w < SAMPLE_THREADS / 32; ++w) { Z += scr[w]; SX += scr[8 + w]; }
            a.stats_out[2 * r] = logf(Z) - SX / Z;
            a.stats_out[2 * r + 1] = 1.0f / Z;
        }
        bar_named(bar_id, SAMPLE_THREADS);
    }

    int choice = bi;
    if (top_k != 1) {
        const float T = ctl.temperature;
        float sc[SAMPLE_EL];
#pragma unroll
        for (int j = 0; j < SAMPLE_EL; ++j) sc[j] = v[j] / T;
        const float smax = bv / T;
        bool keep[SAMPLE_EL];
#pragma unroll
        for (int j = 0; j < SAMPLE_EL; ++j) keep[j] = true;
        if (top_k > 0) {
            // radix select of the top_k-th largest key, 8 bits per pass
            if (tid == 0) { s_prefix = 0u; s_krem = (uint32_t)top_k; }
            uint32_t key[SAMPLE_EL];
#pragma unroll
            for (int j = 0; j < SAMPLE_EL; ++j) key[j] = order_key(sc[j]);
            for (int pass = 0; pass < 4; ++pass) {
                const int shift = 24 - 8 * pass;
                hist[tid] = 0u;
                bar_named(bar_id, SAMPLE_THREADS);
                const uint32_t prefix = s_prefix;
                const uint32_t pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
#pragma unroll
                for (int j = 0; j < SAMPLE_EL; ++j)
                    if ((key[j] & pmask) == prefix) atomicAdd(&hist[(key[j] >> shift) & 255u], 1u);
                bar_named(bar_id, SAMPLE_THREADS);
                if (warp == 0) {
                    // lane covers digits 255-8*lane .. 248-8*lane (descending)
                    uint32_t c8[8], tot = 0u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) { c8[j] = hist[255 - 8 * lane - j]; tot += c8[j]; }
                    uint32_t inc = tot;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
                        if (lane >= o) inc += t;
                    }
                    const uint32_t before = inc - tot, krem = s_krem;
                    if (before < krem && krem <= inc) {
                        uint32_t cum = before;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (cum < krem && krem <= cum + c8[j]) {
                                s_prefix = prefix | ((uint32_t)(255 - 8 * lane - j) << shift);
                                s_krem = krem - cum;
                            }
                            cum += c8[j];
                        }
                    }
                }
                bar_named(bar_id, SAMPLE_THREADS);
            }
            const uint32_t thr = s_prefix;
#pragma unroll
            for (int j = 0; j < SAMPLE_EL; ++j) keep[j] = key[j] >= thr;
        }
        float p[SAMPLE_EL], loc = 0.f;
#pragma unroll
        for (int j = 0; j < SAMPLE_EL; ++j) {
            p[j] = keep[j] ? expf(sc[j] - smax) : 0.f;
            loc += p[j];
        }
        // block exclusive scan of per-thread totals
        float inc = loc;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) s_f[warp] = inc;
        if (tid == 0) { s_pick = 0x7fffffff; s_lastkept = -1; }
        bar_named(bar_id, SAMPLE_THREADS);
        float wbase = 0.f, total = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            if (w < warp) wbase += s_f[w];
            total += s_f[w];
        }
        uint32_t c[4] = {(uint32_t)slot, frame_no, (uint32_t)a.codebook, 0u};
        philox4x32_10(c, ctl.seed_lo, ctl.seed_hi);
        const float u = (float)(c[0] >> 8) * (1.0f / 16777216.0f);
        const float target = u * total;
        float cum = wbase + inc - loc;
        int mine = 0x7fffffff, lastk = -1;
#pragma unroll
        for (int j = 0; j < SAMPLE_EL; ++j) {
            cum += p[j];
            if (keep[j]) {
                lastk = tid * SAMPLE_EL + j;
                if (cum > target && mine == 0x7fffffff) mine = tid * SAMPLE_EL + j;
            }
        }
        if (mine != 0x7fffffff) atomicMin(&s_pick, mine);
        if (lastk >= 0) atomicMax(&s_lastkept, lastk);
        bar_named(bar_id, SAMPLE_THREADS);
        choice = s_pick != 0x7fffffff ? s_pick : s_lastkept;
    }
    if (tid == 0) {
        a.code_cur[r] = choice;
        a.codes_out[(size_t)r * a.Q + a.out_col] = (int64_t)choice;
        if (a.zero_from > 0)
            for (int q = a.zero_from; q < a.Q; ++q) a.codes_out[(size_t)r * a.Q + q] = 0;
        if (is_cb0) {
            if (a.eos_logit && a.eos_prob) a.eos_prob[r] = 1.f / (1.f + expf(-bf2f(a.eos_logit[r])));
            if (ctl.rep_penalty > 1.0f) {
                float* cnt = a.rep_counts + (size_t)slot * CS;
                int W = ctl.rep_window > REP_HIST_MAX ? REP_HIST_MAX : ctl.rep_window;
                if (W > 0) {
                    int head = a.rep_head[slot], filled = a.rep_filled[slot];
                    if (head >= W) head = 0;
                    if (filled >= W) {
                        const int old = a.rep_hist[slot * REP_HIST_MAX + head];
                        cnt[old] -= 1.f;
                        filled = W;
                    } else {
                        filled += 1;
                    }
                    a.rep_hist[slot * REP_HIST_MAX + head] = choice;
                    a.rep_head[slot] = (head + 1) % W;
                    a.rep_filled[slot] = filled;
                }
                cnt[choice] += 1.f;
            }
        }
        if (a.bump_frame) a.frame_ctr[slot] += 1;
    }
    if (a.emb_out) {
        const bf16* e = a.code_emb + ((size_t)(a.emb_p - 1) * CS + choice) * a.emb_rd;
        const bf16* pe = a.pos_emb + (size_t)a.emb_p * a.emb_rd;
        bf16* o = a.emb_out + ((size_t)r * a.emb_row_mul + a.emb_row_add) * a.emb_rd;
        for (int k = tid * 8; k < a.emb_rd; k += SAMPLE_THREADS * 8) {
            float x[8], c[8], sum[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(e + k)), x);
            unpack8(__ldg(reinterpret_cast<const uint4*>(pe + k)), c);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] = x[j] + c[j];
            *reinterpret_cast<uint4*>(o + k) = pack8(sum);
        }
    }
    return choice;
}

static __global__ void __launch_bounds__(SAMPLE_THREADS) k_sample(SampleArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ SampleSmem S_;
    sample_row(a, blockIdx.x, threadIdx.x, S_, 0);
}

}  // namespace vuib
