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
//  * one tcgen05.mma of this shape costs ~96 ns whatever the batch, i.e. an SM consumes weights at
//    only ~42 GB/s, so the K dimension is split over enough CTAs to occupy every SM; the CTAs of a
//    tile (all resident: the grid never exceeds the SM count times two) publish their partial tile,
//    meet on a counter with a bounded wait, and EACH adds the splits - in index order, so the result
//    is deterministic - for its own 1/splits slice of the rows and runs the epilogue functor there
//    (RoPE + KV append, residual add, SwiGLU, logits);
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
constexpr int TC_MAX_STAGES = 12;     // ring depth is set per launch from the shared memory left
constexpr int TC_EPI_BYTES_PER_M = 256;  // epilogue staging per activation row (128 bf16)
constexpr int FLAG_TC_TIMEOUT = 16;
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;  // default bound of every wait below, in polls (TcArgs::spin_limit)

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

// Bounded wait on a phase parity; returns false after `limit` probes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, unsigned limit) {
    const uint32_t a = smem_u32(bar);
    for (unsigned spins = 0; spins < limit; ++spins) {
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

// 32 consecutive accumulator columns of this thread's TMEM lane in one instruction.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
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
    static constexpr bool STAGED = true;
    // While the MMAs run: RoPE rows [cos,sin] x 64 of every activation row's position -> es[m][128].
    __device__ __forceinline__ void stage(unsigned char* es, int tile, int M, int tid) const {
        if (!rope) return;
        uint4* dst = reinterpret_cast<uint4*>(es);
        for (int i = tid; i < M * 16; i += TC_THREADS) {
            const int m = i >> 4, c = i & 15;
            const int pos = row_slot ? __ldcg(row_pos + m) : pos_base + (m + m_off) % rows_per_b;
            dst[i] = __ldg(reinterpret_cast<const uint4*>(rope + (size_t)pos * HD * 2) + c);
        }
    }
    __host__ __device__ TcEpiQkv shifted(int m) const {
        TcEpiQkv o = *this;
        o.q_out += (size_t)m * q_cols;
        if (row_slot) { o.row_slot += m; o.row_pos += m; }
        o.m_off += m;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*,
                                          const unsigned char* es) const {
        const bool odd = n & 1;
        const bool do_rope = rope && n < q_cols + kv_cols;
        const bool to_cache = n >= q_cols;
        int slot[8], pos[8];
        if (to_cache) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // loads first: they do not depend on one another
                const int m = m0 + j < M ? m0 + j : (M > 0 ? M - 1 : 0);
                if (row_slot) { slot[j] = __ldcg(row_slot + m); pos[j] = __ldcg(row_pos + m); }
                else { slot[j] = (m + m_off) / rows_per_b; pos[j] = pos_base + (m + m_off) % rows_per_b; }
            }
        }
        const __nv_bfloat162* rs = reinterpret_cast<const __nv_bfloat162*>(es);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            float t = rbf(v[j]);
            const float other = __shfl_xor_sync(0xffffffffu, t, 1);
            if (m >= M) continue;
            if (do_rope) {
                const __nv_bfloat162 f = rs[m * 64 + (n & (HD - 1))];
                const float c = __low2float(f), sn = __high2float(f);
                t = odd ? rbf(rbf(t * c) + rbf(other * sn)) : rbf(rbf(t * c) + rbf((-other) * sn));
            }
            const bf16 o = f2bf(t);
            if (!to_cache) q_out[(size_t)m * q_cols + n] = o;
            else if (n < q_cols + kv_cols) k_cache[((size_t)slot[j] * max_seq + pos[j]) * kv_cols + (n - q_cols)] = o;
            else v_cache[((size_t)slot[j] * max_seq + pos[j]) * kv_cols + (n - q_cols - kv_cols)] = o;
        }
    }
};

struct TcEpiResidual {  // x += bf16(acc)
    bf16* x; int N; bf16* tap;
    static constexpr bool PAIRED = false;
    static constexpr bool STAGED = true;
    // While the MMAs run: this tile's slice of the residual stream, x[m][tile*128 .. +128) -> es[m][128].
    __device__ __forceinline__ void stage(unsigned char* es, int tile, int M, int tid) const {
        uint4* dst = reinterpret_cast<uint4*>(es);
        for (int i = tid; i < M * 16; i += TC_THREADS) {
            const int m = i >> 4, c = i & 15;
            dst[i] = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * N + tile * TC_TILE_N) + c);
        }
    }
    __host__ __device__ TcEpiResidual shifted(int m) const {
        TcEpiResidual o = *this;
        o.x += (size_t)m * N;
        if (tap) o.tap += (size_t)m * N;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*,
                                          const unsigned char* es) const {
        const bf16* xs = reinterpret_cast<const bf16*>(es);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m >= M) continue;
            const size_t idx = (size_t)m * N + n;
            const bf16 o = f2bf(bf2f(xs[m * TC_TILE_N + (n & (TC_TILE_N - 1))]) + rbf(v[j]));
            x[idx] = o;
            if (tap) tap[idx] = o;
        }
    }
};

struct TcEpiSwiGLU {    // tile rows 0..63 = w1 rows, 64..127 = w3 rows of the same hidden units
    bf16* act; int F;  // hidden unit of tile row r (< 64) is tile*64 + r
    static constexpr bool PAIRED = true;
    static constexpr bool STAGED = false;
    __host__ __device__ TcEpiSwiGLU shifted(int m) const {
        TcEpiSwiGLU o = *this;
        o.act += (size_t)m * F;
        return o;
    }
    // a1 = the unit's w1 sums, a3 = its w3 sums, for activation rows m0..m0+7
    __device__ __forceinline__ void apply_pair(int unit, int m0, int M, const float (&a1)[8],
                                               const float (&a3)[8]) const {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m >= M) continue;
            const float a = rbf(a1[j]), g = rbf(a3[j]);
            const float sl = rbf(a / (1.0f + expf(-a)));
            act[(size_t)m * F + unit] = f2bf(sl * g);
        }
    }
};

struct TcEpiLogits {    // plain bf16 rows (+ optional second copy with its own stride)
    bf16* out; int N; bf16* tap; int tap_stride;
    static constexpr bool PAIRED = false;
    static constexpr bool STAGED = false;
    __host__ __device__ TcEpiLogits shifted(int m) const {
        TcEpiLogits o = *this;
        o.out += (size_t)m * N;
        if (tap) o.tap += (size_t)m * tap_stride;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*,
                                          const unsigned char*) const {
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
    static constexpr bool STAGED = false;
    __host__ __device__ TcEpiProjPos shifted(int m) const {
        TcEpiProjPos o = *this;
        o.out += (size_t)m * row_mul * rd;
        return o;
    }
    __device__ __forceinline__ void apply(int n, int m0, int M, const float (&v)[8], float*,
                                          const unsigned char*) const {
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
    int M, Mpad;      // activation rows in all; rows per CTA padded to a multiple of 16 (<= 256).  M > Mpad: the
                      // grid's z dimension walks blocks of Mpad rows (one launch for a whole prefill)
    int chunks;       // K chunks of 64 in all; split s handles chunks [s*chunks/splits, (s+1)*chunks/splits)
    int stages;       // TMA ring depth (<= TC_MAX_STAGES, <= chunks)
    int splits;       // gridDim.x: 1, 2, 4, 8 or 16 (PAIRED: not 2)
    float* partial;   // (row blocks, tiles, splits, 128, Mpad) fp32 scratch (splits > 1)
    int32_t* counters;  // (2, row blocks x tiles) arrivals / departures, zero between launches
    int tiles;
    int32_t* flag;
    unsigned long long* dbg;  // optional: device-clock stamps of CTA (0,0) (profiling aid)
    unsigned spin_limit;      // polls after which a wait gives up and records FLAG_TC_TIMEOUT
};

__device__ __forceinline__ void tc_stamp(const TcArgs& a, int i) {
    if (a.dbg && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 64) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.dbg[i] = t;
    }
}

template <class Epi>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
          const __grid_constant__ CUtensorMap mapX, TcArgs a, Epi ep_all) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint64_t bar_full[TC_MAX_STAGES], bar_empty[TC_MAX_STAGES], bar_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_bad;
    __shared__ float xchg[Epi::PAIRED ? 128 * 8 : 1];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, tile = blockIdx.y;  // the CTAs of one tile are neighbours in launch order
    const int m_base = blockIdx.z * a.Mpad;           // first activation row of this CTA's block
    const int Mb = min(a.Mpad, a.M - m_base);         // rows of the block
    const int tile_id = blockIdx.z * a.tiles + tile;  // index of the (block, tile) pair in the split-K scratch
    const int all_tiles = gridDim.z * a.tiles;
    const Epi ep = ep_all.shifted(m_base);
    tc_stamp(a, 0);
    const int stages = a.stages;  // <= smallest chunk count of any split
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
    tc_stamp(a, 1);
    // Only now may the next kernel's CTAs become resident: every CTA of this grid already owns its
    // tensor-memory columns, so early dependents can never starve it of them.
    pdl_trigger();

    const int k_first = (int)((long long)split * a.chunks / a.splits);  // in chunks
    const int n_chunks = (int)((long long)(split + 1) * a.chunks / a.splits) - k_first;
    // weight rows of this tile: PAIRED -> 64 rows of each matrix at unit offset tile*64
    const int rowA0 = a.row_off + (Epi::PAIRED ? tile * 64 : tile * TC_TILE_N);
    const int rowA1 = a.row_off + (Epi::PAIRED ? tile * 64 : tile * TC_TILE_N + 64);

    // Roles are per warp: the 31 idle lanes of a role's warp park at __syncwarp(), not in an
    // mbarrier wait, so they cannot hold back the lane that feeds the pipeline.
    if (warp == 0) {
      if (lane == 0) {
        // ---- TMA producer.  Weights for the first ring pass go out before the dependency wait.
        for (int c = 0; c < stages; ++c) {
            unsigned char* st = base + (size_t)c * stage_bytes;
            mbar_expect_tx(&bar_full[c], a_bytes + b_bytes);
            tma_load_2d(st, &mapA0, (k_first + c) * TC_KCHUNK, rowA0, &bar_full[c]);
            tma_load_2d(st + a_bytes / 2, &mapA1, (k_first + c) * TC_KCHUNK, rowA1, &bar_full[c]);
        }
        pdl_wait();
        for (int c = 0; c < stages; ++c)
            tma_load_2d(base + (size_t)c * stage_bytes + a_bytes, &mapX, (k_first + c) * TC_KCHUNK, m_base, &bar_full[c]);
        for (int c = stages; c < n_chunks; ++c) {
            const int s = c % stages;
            if (!mbar_wait(&bar_empty[s], ((c / stages) & 1) ^ 1, 4 * a.spin_limit)) { s_bad = 1; break; }
            unsigned char* st = base + (size_t)s * stage_bytes;
            mbar_expect_tx(&bar_full[s], a_bytes + b_bytes);
            tma_load_2d(st, &mapA0, (k_first + c) * TC_KCHUNK, rowA0, &bar_full[s]);
            tma_load_2d(st + a_bytes / 2, &mapA1, (k_first + c) * TC_KCHUNK, rowA1, &bar_full[s]);
            tma_load_2d(st + a_bytes, &mapX, (k_first + c) * TC_KCHUNK, m_base, &bar_full[s]);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc = umma_idesc_bf16(a.Mpad);
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c % stages;
            if (!mbar_wait(&bar_full[s], (c / stages) & 1, 4 * a.spin_limit)) { s_bad = 1; break; }
            if (a.dbg && split == 0 && tile == 0 && c < 8) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                a.dbg[8 + c] = t;  // when chunk c (< 8) became available to the MMA thread
            }
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
      __syncwarp();
    }
    pdl_wait();
    tc_stamp(a, 2);
    unsigned char* es = base + (size_t)stages * stage_bytes;  // epilogue staging, filled while the MMAs run
    if constexpr (Epi::STAGED) ep.stage(es, tile, Mb, tid);
    // ---- everyone: wait for the accumulator
    const bool done_ok = mbar_wait(&bar_done, 0, 4 * a.spin_limit);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if ((!done_ok || s_bad) && tid == 0) atomicOr(a.flag, FLAG_TC_TIMEOUT);
    tc_stamp(a, 3);

    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);  // thread tid reads tile row tid (TMEM lane)
    if (a.splits == 1) {
        for (int m0 = 0; m0 < a.Mpad; m0 += 8) {
            float v[8];
            tmem_ld8(trow + m0, v);
            if constexpr (Epi::PAIRED) {  // rows r and r+64 are the w1 / w3 sums of hidden unit tile*64 + r
#pragma unroll
                for (int j = 0; j < 8; ++j) xchg[tid * 8 + j] = v[j];
                __syncthreads();
                if (tid < 64) {
                    float g[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) g[j] = xchg[(tid + 64) * 8 + j];
                    ep.apply_pair(tile * 64 + tid, m0, Mb, v, g);
                }
                __syncthreads();
            } else {
                ep.apply(tile * TC_TILE_N + tid, m0, Mb, v, xchg, es);
            }
        }
    } else {
        // partial tile to scratch as [m][n]: the 128 threads of a CTA write 512 contiguous bytes per m
        float* mine = a.partial + ((size_t)tile_id * a.splits + split) * a.Mpad * TC_TILE_N;
        int m0 = 0;
        for (; m0 + 32 <= a.Mpad; m0 += 32) {
            float v[32];
            tmem_ld32(trow + m0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) mine[(size_t)(m0 + j) * TC_TILE_N + tid] = v[j];
        }
        for (; m0 < a.Mpad; m0 += 8) {
            float v[8];
            tmem_ld8(trow + m0, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) mine[(size_t)(m0 + j) * TC_TILE_N + tid] = v[j];
        }
        tc_stamp(a, 4);
        __syncthreads();  // orders every thread's partial stores before thread 0's release below
        if (tid == 0) {
            // arrive, then wait (bounded) until every split of this tile has published its partial
            asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(a.counters + tile_id) : "memory");
            int v = 0;
            unsigned spins = 0;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(a.counters + tile_id) : "memory");
                if (v >= a.splits) break;
                if (++spins > a.spin_limit) { atomicOr(a.flag, FLAG_TC_TIMEOUT); break; }
            }
        }
        __syncthreads();
        tc_stamp(a, 5);
        // This CTA finishes 128/splits rows of the tile: thread = (row j of the slice, column group mg).
        const int rpc = TC_TILE_N / a.splits;       // rows per CTA
        const int j_row = tid % rpc, mg = tid / rpc;  // mg in [0, splits)
        int row;                                      // row inside the tile
        if constexpr (Epi::PAIRED) {
            const int half = rpc / 2;                 // w1 rows, then the matching w3 rows (same warp)
            row = j_row < half ? split * half + j_row : 64 + split * half + (j_row - half);
        } else {
            row = split * rpc + j_row;
        }
        const float* all = a.partial + (size_t)tile_id * a.splits * a.Mpad * TC_TILE_N + row;
        const size_t split_stride = (size_t)a.Mpad * TC_TILE_N;
        const int n_mchunks = a.Mpad / 8;
        for (int chunk0 = 0; chunk0 < n_mchunks; chunk0 += a.splits) {  // uniform trip count: the
            const bool active = chunk0 + mg < n_mchunks;                // epilogues shuffle within a warp
            const int m0 = (active ? chunk0 + mg : n_mchunks - 1) * 8;
            const int Meff = active ? Mb : 0;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int s0 = 0; s0 < a.splits; s0 += 8) {  // up to 64 loads in flight, summed in split order
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
            if constexpr (Epi::PAIRED) {
                const int half = rpc / 2;
                float g[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] = __shfl_xor_sync(0xffffffffu, v[j], half);
                if (j_row < half) ep.apply_pair(tile * 64 + row, m0, Meff, v, g);
            } else {
                ep.apply(tile * TC_TILE_N + row, m0, Meff, v, xchg, es);
            }
        }
        __syncthreads();
        if (tid == 0) {  // the last CTA to leave re-arms both counters for the next launch
            const int old = atomicAdd(a.counters + all_tiles + tile_id, 1);
            if (old == a.splits - 1) {
                a.counters[tile_id] = 0;
                a.counters[all_tiles + tile_id] = 0;
            }
        }
    }
    tc_stamp(a, 6);
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
    const int r = blockIdx.x;
    __shared__ float red[4];
    const bf16* xr = x + ((size_t)r * row_mul + row_add) * K;
    if (K <= 128 * 8) {
        // one 16-byte piece per thread: the row stays in registers between the two passes and the
        // norm weights (constants) are fetched before the predecessor is waited for
        const int k = threadIdx.x * 8;
        const bool on = k < K;
        const uint4 wv = on ? __ldg(reinterpret_cast<const uint4*>(w + k)) : make_uint4(0, 0, 0, 0);
        pdl_wait();
        float f[8], wf[8], o[8];
        unpack8(on ? __ldcg(reinterpret_cast<const uint4*>(xr + k)) : make_uint4(0, 0, 0, 0), f);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        const float rinv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)K + eps);
        if (on) {
            unpack8(wv, wf);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rbf(f[j] * rinv) * wf[j];
            *reinterpret_cast<uint4*>(out + (size_t)r * K + k) = pack8(o);
        }
        return;
    }
    pdl_wait();
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
