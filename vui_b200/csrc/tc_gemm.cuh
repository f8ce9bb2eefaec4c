// Skinny GEMM for many streams / prefill rows on the 5th-generation tensor cores:
//   D[n][m] = sum_k W[n][k] * X[m][k]      (W: weights (N, K) bf16; X: activations (M, K) bf16)
// "swap-AB": a tile of 128 weight rows is the MMA's M side, the (padded) batch of 16..256
// activation rows its N side, so one tcgen05.mma covers every stream at once and each weight
// byte is read from HBM exactly once per step.
//
//  * operands reach shared memory through TMA (cp.async.bulk.tensor.2d, 128-byte swizzle,
//    K-major), one elected thread issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32), the
//    accumulator tile lives in tensor memory and is read back with tcgen05.ld for the epilogue;
//  * an mbarrier ring (full / empty per stage) decouples the TMA thread from the MMA thread; every
//    wait is bounded and records FLAG_TC_TIMEOUT instead of hanging;
//  * the grid is (weight tiles) x (K splits) so that ~all SMs stream weights even when N is small;
//    split partial tiles go to scratch and the LAST CTA to finish a tile adds them in split order
//    (deterministic) and runs the epilogue functor (RoPE + KV append, residual add, SwiGLU, logits);
//  * launched with programmatic dependent launch: the weight tiles of the first stages are
//    requested before the kernel waits for its predecessor, the activations after.
// No TMA load here uses cluster multicast.
#pragma once
#include <cuda.h>

#include "decode_kernels.cuh"

namespace vuib {

constexpr int TC_THREADS = 128;
constexpr int TC_TILE_N = 128;      // weight rows per CTA (two TMA boxes of 64 rows)
constexpr int TC_KCHUNK = 64;       // bf16 per row per stage = 128 bytes = one swizzle span
constexpr int TC_MAX_STAGES = 4;
constexpr int FLAG_TC_TIMEOUT = 16;
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// Bounded wait on a phase parity; returns false after TC_SPIN_LIMIT probes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    const uint32_t a = smem_u32(bar);
    for (unsigned spins = 0; spins < TC_SPIN_LIMIT; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// K-major, 128-byte-swizzled operand tile: rows are 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(smem_tile) >> 4) & 0x3FFF);  // start address
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
    return d;
}

// kind::f16 instruction descriptor: bf16 A and B, fp32 accumulate, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// ---------------------------------------------------------------------------
// Epilogue functors.  A thread owns weight row n (0..127 of the tile) and is handed
// 8 consecutive activation rows m0..m0+7 at a time (the whole CTA calls together).
// ---------------------------------------------------------------------------
struct TcEpiQkv {      // RoPE on q,k + K/V append (EpiQkv of the GEMV path)
    bf16* q_out; int q_cols, kv_cols;
    bf16* k_cache; bf16* v_cache;
    const int32_t* row_slot; const int32_t* row_pos; int max_seq;
    const bf16* rope;
    int rows_per_b, pos_base;
    int m_off;  // row index of m = 0 in the depth-transformer addressing
    static constexpr bool PAIRED = false;
    TcEpiQkv shifted(int m) const {
        TcEpiQkv o = *this;
        o.q_out += (size_t)m * q_cols;
        if (row_slot) { o.row_slot += m; o.row_pos += m; }
        o.m_off += m;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*) const {
        const bool odd = n & 1;
        const bool do_rope = rope && n < q_cols + kv_cols;
        int slot[8], pos[8];
        float c[8], sn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // all loads first: they do not depend on one another
            const int m = m0 + j < M ? m0 + j : (M > 0 ? M - 1 : 0);
            if (row_slot) { slot[j] = __ldcg(row_slot + m); pos[j] = __ldcg(row_pos + m); }
            else { slot[j] = (m + m_off) / rows_per_b; pos[j] = pos_base + (m + m_off) % rows_per_b; }
        }
        if (do_rope) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __nv_bfloat162 f = *reinterpret_cast<const __nv_bfloat162*>(
                    rope + ((size_t)pos[j] * HD + (n & (HD - 1))) * 2);
                c[j] = __low2float(f);
                sn[j] = __high2float(f);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            float t = rbf(v[j]);
            const float other = __shfl_xor_sync(0xffffffffu, t, 1);
            if (m >= M) continue;
            if (do_rope) t = odd ? rbf(rbf(t * c[j]) + rbf(other * sn[j])) : rbf(rbf(t * c[j]) + rbf((-other) * sn[j]));
            const bf16 o = f2bf(t);
            if (n < q_cols) q_out[(size_t)m * q_cols + n] = o;
            else if (n < q_cols + kv_cols) k_cache[((size_t)slot[j] * max_seq + pos[j]) * kv_cols + (n - q_cols)] = o;
            else v_cache[((size_t)slot[j] * max_seq + pos[j]) * kv_cols + (n - q_cols - kv_cols)] = o;
        }
    }
};

struct TcEpiResidual {  // x += bf16(acc)
    bf16* x; int N; bf16* tap;
    static constexpr bool PAIRED = false;
    TcEpiResidual shifted(int m) const {
        TcEpiResidual o = *this;
        o.x += (size_t)m * N;
        if (tap) o.tap += (size_t)m * N;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*) const {
        unsigned short xb[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)  // the 8 residual values are fetched together, then added and stored
            xb[j] = (m0 + j < M) ? __ldcg(reinterpret_cast<const unsigned short*>(x) + (size_t)(m0 + j) * N + n) : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m >= M) continue;
            const size_t idx = (size_t)m * N + n;
            const bf16 o = f2bf(bf2f(__ushort_as_bfloat16(xb[j])) + rbf(v[j]));
            x[idx] = o;
            if (tap) tap[idx] = o;
        }
    }
};

struct TcEpiSwiGLU {    // tile rows 0..63 = w1 rows, 64..127 = w3 rows of the same hidden units
    bf16* act; int F;  // hidden unit of tile row r (< 64) is tile*64 + r
    static constexpr bool PAIRED = true;
    TcEpiSwiGLU shifted(int m) const {
        TcEpiSwiGLU o = *this;
        o.act += (size_t)m * F;
        return o;
    }
    __device__ __forceinline__ void apply(int n_global_unit, int r_local, int m0, int M, const float (&v)[8],
                                          float* xchg /* [128][8] */) const {
#pragma unroll
        for (int j = 0; j < 8; ++j) xchg[r_local * 8 + j] = v[j];
        __syncthreads();
        if (r_local < 64) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int m = m0 + j;
                if (m >= M) continue;
                const float a = rbf(v[j]), g = rbf(xchg[(r_local + 64) * 8 + j]);
                const float s = rbf(a / (1.0f + expf(-a)));
                act[(size_t)m * F + n_global_unit] = f2bf(s * g);
            }
        }
        __syncthreads();
    }
};

struct TcEpiLogits {    // plain bf16 rows (+ optional second copy with its own stride)
    bf16* out; int N; bf16* tap; int tap_stride;
    static constexpr bool PAIRED = false;
    TcEpiLogits shifted(int m) const {
        TcEpiLogits o = *this;
        o.out += (size_t)m * N;
        if (tap) o.tap += (size_t)m * tap_stride;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*) const {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m >= M) continue;
            const bf16 o = f2bf(v[j]);
            out[(size_t)m * N + n] = o;
            if (tap) tap[(size_t)m * tap_stride + n] = o;
        }
    }
};

struct TcEpiProjPos {   // depth position 0: bf16(acc) + pos_emb[0], written to row m*row_mul
    const bf16* pos_emb; bf16* out; int rd, row_mul;
    static constexpr bool PAIRED = false;
    TcEpiProjPos shifted(int m) const {
        TcEpiProjPos o = *this;
        o.out += (size_t)m * row_mul * rd;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*) const {
        const float pe = bf2f(pos_emb[n]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m >= M) continue;
            out[(size_t)m * row_mul * rd + n] = f2bf(rbf(v[j]) + pe);
        }
    }
};

struct TcArgs {
    int N;            // weight rows, a multiple of 128 (PAIRED: hidden units, a multiple of 64)
    int row_off;      // first weight row of tile 0 inside the mapped matrix (stacked depth heads)
    int M, Mpad;      // activation rows, padded to a multiple of 16 (<= 256)
    int chunks;       // K chunks of 64 handled by one CTA
    int splits;       // gridDim.y
    float* partial;   // (tiles, splits, 128, Mpad) fp32 scratch (splits > 1)
    int32_t* counters;  // (tiles) zero between launches
    int32_t* flag;
};

template <class Epi>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
          const __grid_constant__ CUtensorMap mapX, TcArgs a, Epi ep) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint64_t bar_full[TC_MAX_STAGES], bar_empty[TC_MAX_STAGES], bar_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_last, s_bad;
    __shared__ float xchg[Epi::PAIRED ? 128 * 8 : 1];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int stages = a.chunks < TC_MAX_STAGES ? a.chunks : TC_MAX_STAGES;
    const uint32_t a_bytes = TC_TILE_N * TC_KCHUNK * 2, b_bytes = (uint32_t)a.Mpad * TC_KCHUNK * 2;
    const uint32_t stage_bytes = a_bytes + ((b_bytes + 1023u) & ~1023u);
    unsigned char* base = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
        mbar_init(&bar_done, 1);
        s_bad = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    int tmem_cols = 32;
    while (tmem_cols < a.Mpad) tmem_cols <<= 1;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // Only now may the next kernel's CTAs become resident: every CTA of this grid already owns its
    // tensor-memory columns, so early dependents can never starve it of them.
    pdl_trigger();

    const int k_first = split * a.chunks;  // in chunks
    // weight rows of this tile: PAIRED -> 64 rows of each matrix at unit offset tile*64
    const int rowA0 = a.row_off + (Epi::PAIRED ? tile * 64 : tile * TC_TILE_N);
    const int rowA1 = a.row_off + (Epi::PAIRED ? tile * 64 : tile * TC_TILE_N + 64);

    if (warp == 0 && lane == 0) {
        // ---- TMA producer.  Weights for the first ring pass go out before the dependency wait.
        for (int c = 0; c < stages; ++c) {
            unsigned char* st = base + (size_t)c * stage_bytes;
            mbar_expect_tx(&bar_full[c], a_bytes + b_bytes);
            tma_load_2d(st, &mapA0, (k_first + c) * TC_KCHUNK, rowA0, &bar_full[c]);
            tma_load_2d(st + a_bytes / 2, &mapA1, (k_first + c) * TC_KCHUNK, rowA1, &bar_full[c]);
        }
        pdl_wait();
        for (int c = 0; c < stages; ++c)
            tma_load_2d(base + (size_t)c * stage_bytes + a_bytes, &mapX, (k_first + c) * TC_KCHUNK, 0, &bar_full[c]);
        for (int c = stages; c < a.chunks; ++c) {
            const int s = c % stages;
            if (!mbar_wait(&bar_empty[s], ((c / stages) & 1) ^ 1)) { s_bad = 1; break; }
            unsigned char* st = base + (size_t)s * stage_bytes;
            mbar_expect_tx(&bar_full[s], a_bytes + b_bytes);
            tma_load_2d(st, &mapA0, (k_first + c) * TC_KCHUNK, rowA0, &bar_full[s]);
            tma_load_2d(st + a_bytes / 2, &mapA1, (k_first + c) * TC_KCHUNK, rowA1, &bar_full[s]);
            tma_load_2d(st + a_bytes, &mapX, (k_first + c) * TC_KCHUNK, 0, &bar_full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc = umma_idesc_bf16(a.Mpad);
        for (int c = 0; c < a.chunks; ++c) {
            const int s = c % stages;
            if (!mbar_wait(&bar_full[s], (c / stages) & 1)) { s_bad = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* st = base + (size_t)s * stage_bytes;
            const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + a_bytes);
#pragma unroll
            for (int kk = 0; kk < TC_KCHUNK / 16; ++kk)  // 16 bf16 = 32 bytes = 2 descriptor units per step
                umma_bf16(tmem, da + 2 * kk, db + 2 * kk, idesc, (c > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&bar_empty[s]);
        }
        umma_commit(&bar_done);
    }
    if (warp != 0 || lane != 0) pdl_wait();
    // ---- everyone: wait for the accumulator
    const bool done_ok = mbar_wait(&bar_done, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if ((!done_ok || s_bad) && tid == 0) atomicOr(a.flag, FLAG_TC_TIMEOUT);

    const int r_local = tid;                                   // tile row = TMEM lane
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    const int n_global = Epi::PAIRED ? tile * 64 + (r_local & 63) : tile * TC_TILE_N + r_local;

    if (a.splits == 1) {
        for (int m0 = 0; m0 < a.Mpad; m0 += 8) {
            float v[8];
            tmem_ld8(trow + m0, v);
            if constexpr (Epi::PAIRED) ep.apply(n_global, r_local, m0, a.M, v, xchg);
            else ep.apply(n_global, m0, a.M, v, xchg);
        }
    } else {
        // partial tile to scratch as [m][n]: the 128 threads of a CTA write 512 contiguous bytes per m
        float* mine = a.partial + ((size_t)tile * a.splits + split) * a.Mpad * TC_TILE_N;
        for (int m0 = 0; m0 < a.Mpad; m0 += 8) {
            float v[8];
            tmem_ld8(trow + m0, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) mine[(size_t)(m0 + j) * TC_TILE_N + r_local] = v[j];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int old = atomicAdd(a.counters + tile, 1);
            s_last = (old == a.splits - 1);
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            // The last CTA of the tile adds the splits in index order.  Thread n keeps its row: for
            // every (split, m) the 128 threads read 512 contiguous bytes; 8 rows x up to 8 splits of
            // loads are in flight before the first add.
            const float* all = a.partial + (size_t)tile * a.splits * a.Mpad * TC_TILE_N + r_local;
            const size_t split_stride = (size_t)a.Mpad * TC_TILE_N;
            for (int m0 = 0; m0 < a.Mpad; m0 += 8) {
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int s0 = 0; s0 < a.splits; s0 += 8) {
                    float p[8][8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            p[u][j] = (s0 + u < a.splits)
                                          ? __ldcg(all + (size_t)(s0 + u) * split_stride + (size_t)(m0 + j) * TC_TILE_N)
                                          : 0.f;
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] += p[u][j];
                }
                if constexpr (Epi::PAIRED) ep.apply(n_global, r_local, m0, a.M, v, xchg);
                else ep.apply(n_global, m0, a.M, v, xchg);
            }
            if (tid == 0) a.counters[tile] = 0;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Row-wise helpers of the batched path.
// ---------------------------------------------------------------------------

// xn[r] = RMSNorm(x[r*row_mul + row_add]) * w   (bf16 rounding as StageNorm)
__global__ void __launch_bounds__(128) k_rmsnorm_rows(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                      float eps, bf16* __restrict__ out, int K, int row_mul,
                                                      int row_add) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    __shared__ float red[4];
    const bf16* xr = x + ((size_t)r * row_mul + row_add) * K;
    float ss = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += 128 * 8) {
        float f[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(xr + k)), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float rinv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)K + eps);
    for (int k = threadIdx.x * 8; k < K; k += 128 * 8) {
        float f[8], wf[8], o[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(xr + k)), f);
        unpack8(__ldg(reinterpret_cast<const uint4*>(w + k)), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rbf(f[j] * rinv) * wf[j];
        *reinterpret_cast<uint4*>(out + (size_t)r * K + k) = pack8(o);
    }
}

// Depth-transformer attention for many rows: one CTA per row, one warp per head
// (the same arithmetic as StageRqAttn, written to a buffer instead of a GEMV tile).
__global__ void __launch_bounds__(256) k_rq_attn_rows(StageRqAttn st, bf16* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    // stage<512>() writes row rr of a tile at Xs + rr*K: aim tile row 0 at this row's output
    st.template stage<512>(out + (size_t)blockIdx.x * 512, blockIdx.x, 1);
}

// eos_head for many rows: one warp per row (Linear with bias, model.py:1099).
__global__ void __launch_bounds__(128) k_eos_rows(const bf16* __restrict__ hidden, const bf16* __restrict__ w,
                                                  const bf16* __restrict__ b, bf16* __restrict__ out, int M, int K) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= M) return;
    float acc = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        float x[8], wf[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(hidden + (size_t)r * K + k)), x);
        unpack8(__ldg(reinterpret_cast<const uint4*>(w + k)), wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(wf[j], x[j], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[r] = f2bf(acc + bf2f(b[0]));
}

}  // namespace vuib
