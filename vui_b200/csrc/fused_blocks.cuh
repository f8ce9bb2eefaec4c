// One transformer layer of a single-row decode step in TWO kernels instead of five.
//
// A chain of dependent launches costs ~3 us per hand-over whatever the bytes, so the number of
// hand-overs is what a one-stream frame pays for.  Both kernels here run as thread-block clusters of
// 8 CTAs (the portable size: this part's GPCs do not all hold 16 free SMs); what used to cross a kernel boundary (q/k/v -> attention -> out_proj; SwiGLU -> w2) now
// crosses a hardware cluster barrier through distributed shared memory, and only the residual stream
// crosses launches, as per-cluster partial rows that the consumer adds in a fixed order:
//
//   k_attn_block  (one cluster per kv head)   x = x_in + bf16(sum parts_in); h = RMSNorm(x);
//       this head group's Wqkv rows (+RoPE, K/V append) -> cluster exchange -> attention over the
//       cache, keys split over the 8 CTAs, partial softmax states exchanged and merged in CTA order
//       -> this head group's K-slice of out_proj -> parts_out[kv head][d]      (fp32 partial rows)
//   k_mlp_block   (11 or 12 clusters)         x = x_in + bf16(sum parts_in); h = RMSNorm(x);
//       a slice of w1/w3 rows -> SiLU*gate -> cluster exchange -> the matching K-slice of w2
//       -> parts_out[cluster][d]
//
// Rounding points are those of the five-kernel path (every tensor PyTorch materialises in bf16 is
// rounded at the same place: src/vui/model.py:204-297, 359-375; src/vui/rope.py:50); out_proj and w2
// sums are accumulated as per-cluster partials in fp32 and rounded once, so only the fp32 summation
// order differs.
//
// Weights reach shared memory through bulk asynchronous copies (cp.async.bulk + mbarrier) issued
// BEFORE the kernel waits for its predecessor (programmatic dependent launch): the copy engine keeps
// HBM busy across the hand-over whenever both kernels fit on an SM together (the column slices of out_proj
// and w2 come as one tiled copy each: a row-by-row series of small bulk copies measured ~30 ns apiece); each kernel also asks the
// L2 for its successor's matrices, so that a successor that could not start early still finds them on
// chip.  No copy here uses cluster multicast.  Every mbarrier wait is
// bounded; cluster barriers are reached by every CTA unconditionally.
#pragma once
#include <cooperative_groups.h>

#include "tc_gemm.cuh"  // smem_u32, mbarrier helpers

namespace vuib {

namespace cg = cooperative_groups;

constexpr int FB_THREADS = 256;  // attention block
constexpr int FB_WARPS = 8;
constexpr int FB_CL = 8;         // CTAs per cluster
constexpr int FB_HINT_CLUSTERS = 6;   // clusters of an MLP block that issue the K/V hints (those resident early)
constexpr int FB_ATT_PRE = 4;    // key blocks (of 32 per CTA) whose loads are in flight before use
constexpr int FB_MAX_PF = 3;     // matrices of the successor a kernel asks the L2 for

// Regions of constant memory (the next kernel's matrices) to pull into L2, shared by the whole grid.
struct PrefetchList {
    const void* ptr[FB_MAX_PF];
    unsigned long long bytes[FB_MAX_PF];
};

__device__ __forceinline__ void prefetch_l2(const PrefetchList& pf, int n_threads_cta) {
    const size_t tid = (size_t)blockIdx.x * n_threads_cta + threadIdx.x, nth = (size_t)gridDim.x * n_threads_cta;
#pragma unroll
    for (int r = 0; r < FB_MAX_PF; ++r) {
        if (!pf.ptr[r]) continue;
        const char* base = static_cast<const char*>(pf.ptr[r]);
        const size_t lines = (size_t)pf.bytes[r] / 128;
        for (size_t i = tid; i < lines; i += nth) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + i * 128));
    }
}
// Split cluster barrier: arrive when the CTA starts, wait right before the first access to a peer's
// shared memory, which is only legal once every CTA of the cluster has started.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
// After fence.mbarrier_init.release.cluster has published the CTA's mbarriers, the arrival itself needs no release.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ void fb_stamp(unsigned long long* dbg, int i) {
    if (dbg && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        dbg[i] = t;
    }
}

// One-way exchange inside a cluster: a value is stored into a peer's shared memory and, in the same
// operation, counted on an mbarrier of that peer (st.async ... mbarrier::complete_tx::bytes).  The
// receiver arms its mbarrier with the number of bytes all peers will send and waits for the phase: one
// hop, where a cluster barrier costs an arrive, the barrier itself and a wait.  Receivers cannot retire
// before everything addressed to them has landed, and senders only address peers that still wait.
__device__ __forceinline__ uint32_t peer_addr(const void* local_smem, int peer_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local_smem)), "r"(peer_rank));
    return r;
}
__device__ __forceinline__ void push_f32(uint32_t dst, uint32_t bar, float v) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
                 ::"r"(dst), "f"(v), "r"(bar) : "memory");
}
__device__ __forceinline__ void push_f32x2(uint32_t dst, uint32_t bar, float v0, float v1) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
                 ::"r"(dst), "f"(v0), "f"(v1), "r"(bar) : "memory");
}
// Bounded wait for everything peers send to this CTA's mbarrier (phase 0), with cluster-scope acquire.
__device__ __forceinline__ bool wait_pushed(uint64_t* bar, unsigned limit) {
    const uint32_t a = smem_u32(bar);
    for (unsigned spins = 0; spins < limit; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], 0;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a)
            : "memory");
        if (ok) return true;
    }
    return false;
}

constexpr int FLAG_COPY_TIMEOUT = 16;  // same bit as the tensor-core pipeline: "a bounded wait ran out"

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Waits for this CTA's weight copies; on expiry records the flag and waits once more so that the
// CTA does not retire with copies still landing in its shared memory.
__device__ __forceinline__ void wait_weights(uint64_t* bar, unsigned limit, int32_t* flag) {
    if (!mbar_wait(bar, 0, limit)) {
        if (threadIdx.x == 0) atomicOr(flag, FLAG_COPY_TIMEOUT);
        mbar_wait(bar, 0, limit);
    }
}

// x[k] = x_in[k] + bf16(sum_p parts[p][k]) for this thread's EPT consecutive elements.  All rows (at
// most FB_MAX_PARTS) are requested at once and added in row order.
constexpr int FB_MAX_PARTS = 16;
template <int K, int EPT>
__device__ __forceinline__ void load_residual(const bf16* x_in, const float* parts, int n_parts, int k0,
                                              float (&x)[EPT]) {
    static_assert(EPT == 2 || EPT == 4, "2 or 4 elements per thread");
    float s[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) s[j] = 0.f;
    if constexpr (EPT == 4) {
        const uint2 xr = __ldcg(reinterpret_cast<const uint2*>(x_in + k0));
        float4 p[FB_MAX_PARTS];
#pragma unroll
        for (int u = 0; u < FB_MAX_PARTS; ++u)
            p[u] = u < n_parts ? __ldcg(reinterpret_cast<const float4*>(parts + (size_t)u * K + k0))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < FB_MAX_PARTS; ++u) { s[0] += p[u].x; s[1] += p[u].y; s[2] += p[u].z; s[3] += p[u].w; }
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&xr);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    } else {
        const unsigned xr = __ldcg(reinterpret_cast<const unsigned*>(x_in + k0));
        float2 p[FB_MAX_PARTS];
#pragma unroll
        for (int u = 0; u < FB_MAX_PARTS; ++u)
            p[u] = u < n_parts ? __ldcg(reinterpret_cast<const float2*>(parts + (size_t)u * K + k0)) : make_float2(0.f, 0.f);
#pragma unroll
        for (int u = 0; u < FB_MAX_PARTS; ++u) { s[0] += p[u].x; s[1] += p[u].y; }
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr));
        x[0] = a.x; x[1] = a.y;
    }
    if (n_parts > 0) {
#pragma unroll
        for (int j = 0; j < EPT; ++j) x[j] = rbf(x[j] + rbf(s[j]));
    }
}

template <int EPT>
__device__ __forceinline__ void store_bf16(bf16* dst, const float (&x)[EPT]) {
    if constexpr (EPT == 4) {
        uint2 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
        h[0] = __floats2bfloat162_rn(x[0], x[1]);
        h[1] = __floats2bfloat162_rn(x[2], x[3]);
        *reinterpret_cast<uint2*>(dst) = u;
    } else {
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(x[0], x[1]);
    }
}

// RMSNorm of the CTA's copy of x (thread holds EPT elements) into shared memory as bf16.
template <int K, int EPT, int NW>
__device__ __forceinline__ void norm_to_smem(const float (&x)[EPT], const float (&w)[EPT], float eps, bf16* xs, int k0,
                                             float* red) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPT; ++j) ss = fmaf(x[j], x[j], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < NW; ++i) tot += red[i];
    const float rinv = rsqrtf(tot / (float)K + eps);
    float o[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) o[j] = rbf(x[j] * rinv) * w[j];
    store_bf16<EPT>(xs + k0, o);
}

// This lane's share of the normed row: K / 256 sixteen-byte pieces, as floats.
template <int K>
__device__ __forceinline__ void load_h(const bf16* xs, float (&hf)[K / 32], int lane) {
#pragma unroll
    for (int it = 0; it < K / 256; ++it) {
        float t[8];
        unpack8(*reinterpret_cast<const uint4*>(xs + it * 256 + lane * 8), t);
#pragma unroll
        for (int j = 0; j < 8; ++j) hf[it * 8 + j] = t[j];
    }
}

// NR dot products of weight rows in shared memory with the normed row, this lane's share of each.
// Every load is issued before the first use and every row has two accumulators of its own, so the
// dependent chains are short and many.
template <int K, int NR>
__device__ __forceinline__ void dot_rows(const bf16* const (&wrow)[NR], const float (&hf)[K / 32], int lane,
                                         float (&acc)[NR]) {
    constexpr int IT = K / 256;
    uint4 w[NR][IT];
#pragma unroll
    for (int i = 0; i < NR; ++i)
#pragma unroll
        for (int it = 0; it < IT; ++it) w[i][it] = *reinterpret_cast<const uint4*>(wrow[i] + it * 256 + lane * 8);
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            float wf[8];
            unpack8(w[i][it], wf);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a0 = fmaf(wf[j], hf[it * 8 + j], a0);
                a1 = fmaf(wf[4 + j], hf[it * 8 + 4 + j], a1);
            }
        }
        acc[i] = a0 + a1;
    }
}

// NROWS dot products of weight rows in shared memory (row-major, K bf16 each, rows contiguous) with the
// normed row xs (bf16) on the tensor cores: mma.sync m16n8k16, weight rows as the M side, K split over
// the CTA's NW warps.  A dot product does not care in which order k is visited, so
//  * a thread feeds two k-steps from ONE 16-byte load per row: the 8 consecutive elements
//    [8t, 8t+8) of a 32-element block go to fragment positions {2t,2t+1 | 2t+8,2t+9} of step 0 and of
//    step 1, and the same 8 elements of xs go to the B fragment;
//  * row g of a tile visits the blocks of the warp's slice rotated by g, and column g of the B operand
//    carries xs at that same block, so the two rows served in one shared-memory phase read different
//    banks although their stride is a multiple of 128 bytes; row g's sum is then D[g][g].
// Partial sums land in red[warp][row]; the caller adds them over the warps after a __syncthreads().
template <int K, int NROWS, int NW>
__device__ __forceinline__ void mma_rows(const bf16* rows, const bf16* xs, float* red, int warp, int lane) {
    constexpr int NT = (NROWS + 15) / 16;      // 16-row tiles
    constexpr int NBS = K / 32 / NW;           // 32-element blocks per warp
    static_assert(K % (32 * NW) == 0 && NBS >= 2 && NBS % 2 == 0, "every warp takes an even number of blocks");
    const int g = lane >> 2, t = lane & 3;
    float d[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.f;
#pragma unroll
    for (int i = 0; i < NBS; ++i) {
        const int kb = (warp * NBS + ((i + g) % NBS)) * 32 + 8 * t;
        const uint4 hb = *reinterpret_cast<const uint4*>(xs + kb);
#pragma unroll
        for (int tl = 0; tl < NT; ++tl) {
            const int r0 = min(tl * 16 + g, NROWS - 1), r1 = min(tl * 16 + 8 + g, NROWS - 1);
            const uint4 w0 = *reinterpret_cast<const uint4*>(rows + (size_t)r0 * K + kb);
            const uint4 w1 = *reinterpret_cast<const uint4*>(rows + (size_t)r1 * K + kb);
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(d[tl][0]), "+f"(d[tl][1]), "+f"(d[tl][2]), "+f"(d[tl][3])
                         : "r"(w0.x), "r"(w1.x), "r"(w0.y), "r"(w1.y), "r"(hb.x), "r"(hb.y));
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(d[tl][0]), "+f"(d[tl][1]), "+f"(d[tl][2]), "+f"(d[tl][3])
                         : "r"(w0.z), "r"(w1.z), "r"(w0.w), "r"(w1.w), "r"(hb.z), "r"(hb.w));
        }
    }
    if (t == (g >> 1)) {  // this thread holds D[g][g] and D[g+8][g] of every tile
#pragma unroll
        for (int tl = 0; tl < NT; ++tl) {
            red[warp * (NT * 16) + tl * 16 + g] = (g & 1) ? d[tl][1] : d[tl][0];
            red[warp * (NT * 16) + tl * 16 + 8 + g] = (g & 1) ? d[tl][3] : d[tl][2];
        }
    }
}

// Row r's total after mma_rows: the warps' partial sums in warp order.
template <int NROWS, int NW>
__device__ __forceinline__ float mma_row_total(const float* red, int r) {
    constexpr int NT = (NROWS + 15) / 16;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += red[w * (NT * 16) + r];
    return s;
}

// Sum NV values per lane over a group of lanes (xor offsets O, O/2, ..., 1) with the array halved at
// every step while it has more than one entry: NV - 1 + (rounds left) shuffles instead of NV x rounds.
// Afterwards a lane holds the total of ONE value: the halving round at offset o keeps the upper half of
// the array in lanes whose bit o is set, so its index is made of those bits, most significant first.
template <int NV, int O>
struct GroupReduce {
    static __device__ __forceinline__ float run(const float (&v)[NV], int lane) {
        if constexpr (NV > 1) {
            float k[NV / 2];
            const bool up = (lane & O) != 0;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                const float keep = up ? v[i + NV / 2] : v[i];
                const float send = up ? v[i] : v[i + NV / 2];
                k[i] = keep + __shfl_xor_sync(0xffffffffu, send, O);
            }
            if constexpr (O > 1) return GroupReduce<NV / 2, O / 2>::run(k, lane);
            else return k[0];
        } else {
            const float c[1] = {v[0] + __shfl_xor_sync(0xffffffffu, v[0], O)};
            if constexpr (O > 1) return GroupReduce<1, O / 2>::run(c, lane);
            else return c[0];
        }
    }
    // index of the value this lane ends up with
    static __device__ __forceinline__ int index(int lane) {
        if constexpr (NV > 1) {
            const int bit = (lane & O) ? NV / 2 : 0;
            if constexpr (O > 1) return bit + GroupReduce<NV / 2, O / 2>::index(lane);
            else return bit;
        } else {
            return 0;
        }
    }
};

// Rows of a small matrix in shared memory (row-major, C columns of bf16, C / 8 lanes per row) times a
// vector in shared memory (fp32): the warp's RW rows at once, each lane accumulating NV rows before one
// halving reduction; out[row] is written by the lanes that end up holding a row's total.
template <int C, int RW>
__device__ __forceinline__ void small_matvec(const bf16* mat, const float* vec, int row0, float* out, int lane) {
    constexpr int LPR = (C / 8 < 32) ? C / 8 : 32;   // lanes per row
    constexpr int CPL = C / 8 / LPR;                 // 16-byte pieces per lane and row
    constexpr int RPP = 32 / LPR;                    // rows in flight per pass
    constexpr int NV = RW / RPP;                     // rows accumulated per lane
    static_assert(C % 8 == 0 && (C / 8) % LPR == 0 && RW % RPP == 0 && (NV & (NV - 1)) == 0 && NV <= LPR, "shape");
    const int cl = lane % LPR, grp = lane / LPR;
    float vf[CPL][8];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        const float4 a0 = *reinterpret_cast<const float4*>(vec + (c * LPR + cl) * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(vec + (c * LPR + cl) * 8 + 4);
        vf[c][0] = a0.x; vf[c][1] = a0.y; vf[c][2] = a0.z; vf[c][3] = a0.w;
        vf[c][4] = a1.x; vf[c][5] = a1.y; vf[c][6] = a1.z; vf[c][7] = a1.w;
    }
    uint4 w[NV][CPL];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int c = 0; c < CPL; ++c)
            w[i][c] = *reinterpret_cast<const uint4*>(mat + (size_t)(row0 + grp * NV + i) * C + (c * LPR + cl) * 8);
    float s[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            float wf[8];
            unpack8(w[i][c], wf);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a0 = fmaf(wf[j], vf[c][j], a0);
                a1 = fmaf(wf[4 + j], vf[c][4 + j], a1);
            }
        }
        s[i] = a0 + a1;
    }
    const float tot = GroupReduce<NV, LPR / 2>::run(s, lane);
    constexpr int WRITERS_STRIDE = LPR / NV;  // lanes of a group that differ only in the low bits hold the same row
    if (cl % WRITERS_STRIDE == 0) out[row0 + grp * NV + GroupReduce<NV, LPR / 2>::index(lane)] = tot;
}

// ---------------------------------------------------------------------------
// Attention block
// ---------------------------------------------------------------------------
struct AttnBlockArgs {
    const bf16* x_in;       // (K) residual stream before this layer (or the MLP block's input row)
    const float* parts_in;  // (n_parts_in, K) partial rows of the previous block's last product
    int n_parts_in;
    bf16* x_out;            // (K) x as this block sees it (read by the MLP block that follows)
    bf16* tap;              // optional second copy of x
    const bf16* norm_w;
    float eps;
    const bf16* wqkv;       // ((Hq + 2 Hkv) * 64, K), rows q | k | v
    const bf16* wo;         // (K, Hq * 64)
    float* parts_out;       // (Hkv, K)
    bf16* k_cache;          // (slots, max_seq, Hkv, 64) of this layer
    bf16* v_cache;
    const int32_t* row_slot;  // checked (slot, position) of the row; NULL -> fixed_slot / fixed_pos
    const int32_t* row_pos;
    int fixed_slot, fixed_pos;
    int max_seq, n_slots;
    const bf16* rope;       // (max_seq, 64, 2) or NULL
    int Hq, Hkv;
    int32_t* flag;
    unsigned spin_limit;
    PrefetchList next;      // the following kernel's matrices
    unsigned long long* dbg;  // optional: device-clock stamps of CTA 0 (profiling aid)
};

template <int K, int G>
struct AttnBlockSmem {
    static constexpr int QR = G * HD / FB_CL;  // q rows of this CTA (16 or 8)
    static constexpr int KR = HD / FB_CL;      // k rows, and v rows (8)
    static constexpr int NR = QR + 2 * KR;
    static constexpr int NP = NR / 2;          // interleaved row pairs
    static constexpr int PPW = (NP + FB_WARPS - 1) / FB_WARPS;  // pairs per warp
    static constexpr int OR = K / FB_CL;       // out_proj rows of this CTA
    static constexpr int OC = G * HD;          // out_proj columns (this head group's slice)
    alignas(128) bf16 wo[OR * OC];             // destination of a tiled copy: first, 128-byte aligned
    alignas(16) bf16 w[NR * K];
    alignas(16) bf16 xs[K];
    alignas(16) float qkv[G * HD + 2 * HD];    // q heads | new k | new v of the head group (bf16 values)
    float part[FB_CL][G][HD + 2];              // per CTA: acc[64], m, l
    float wpart[FB_WARPS][G][8][10];           // per warp: [s][acc8, m, l]
    alignas(16) float attn[G * HD];
    float s_new[G];
    float red[FB_WARPS];
    float dots[FB_WARPS * ((NR + 15) / 16) * 16];  // per-warp partial sums of the q/k/v rows
    alignas(8) uint64_t bar;      // weight copies
    alignas(8) uint64_t bar_qkv;  // q/k/v vector complete (all peers' rows)
    alignas(8) uint64_t bar_part; // all peers' partial softmax states
};

// SHORT: the cache holds at most 16 positions (the depth transformer): every CTA attends over all of
// them after the q/k/v exchange, which saves the second exchange.
template <int K, int G, bool SHORT>
__global__ void __launch_bounds__(FB_THREADS, 1) k_attn_block(const __grid_constant__ CUtensorMap map_wo, AttnBlockArgs a) {
    using S = AttnBlockSmem<K, G>;
    static_assert(!SHORT || G == 1, "the short form handles one query head per cluster");
    constexpr int EPT = K / FB_THREADS;
    constexpr int QR = S::QR, KR = S::KR, OR = S::OR, OC = S::OC, NP = S::NP;
    static_assert(NP * FB_CL <= FB_THREADS, "eight threads finish each row pair");
    extern __shared__ __align__(128) unsigned char fb_smem[];
    S& sm = *reinterpret_cast<S*>(fb_smem);
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int kvh = blockIdx.x / FB_CL;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qcols = a.Hq * HD, kvcols = a.Hkv * HD;
    fb_stamp(a.dbg, 0);
    pdl_trigger();

    // ---- weights: bulk copies into shared memory, before the predecessor is waited for
    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&sm.bar, 1);
            mbar_init(&sm.bar_qkv, 1);
            mbar_init(&sm.bar_part, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&sm.bar_qkv, (uint32_t)((G * HD + 2 * HD) * 4));
            mbar_expect_tx(&sm.bar_part, (uint32_t)(FB_CL * G * (HD + 2) * 4));
        }
    }
    __syncthreads();
    // After the mbarriers exist (a peer that has passed cluster_wait() may push to them) and BEFORE the weight copies
    // are issued: with copies of this thread in flight the releasing arrival took as long as the copies (1.3 us), which
    // a cluster that only becomes resident when the previous kernel's CTAs leave pays on the chain.
    cluster_arrive_relaxed();
    if (tid == 0) {
        mbar_expect_tx(&sm.bar, (uint32_t)(S::NR * K * 2 + OR * OC * 2));
        bulk_g2s(sm.w, a.wqkv + (size_t)(kvh * G * HD + rank * QR) * K, QR * K * 2, &sm.bar);
        bulk_g2s(sm.w + QR * K, a.wqkv + (size_t)(qcols + kvh * HD + rank * KR) * K, KR * K * 2, &sm.bar);
        bulk_g2s(sm.w + (QR + KR) * K, a.wqkv + (size_t)(qcols + kvcols + kvh * HD + rank * KR) * K, KR * K * 2, &sm.bar);
        // the out_proj slice (OR rows x OC columns of a row-major matrix) as ONE tiled copy
        tma_load_2d(sm.wo, &map_wo, kvh * OC, rank * OR, &sm.bar);
    }
    prefetch_l2(a.next, FB_THREADS);
    const int k0 = tid * EPT;
    // requested here, converted after the wait (nothing in the prologue waits for a load, see the MLP block)
    alignas(8) bf16 nw_raw[EPT];
    if constexpr (EPT == 4) *reinterpret_cast<uint2*>(nw_raw) = __ldg(reinterpret_cast<const uint2*>(a.norm_w + k0));
    else *reinterpret_cast<unsigned*>(nw_raw) = __ldg(reinterpret_cast<const unsigned*>(a.norm_w + k0));
    // ---- the row's old keys and its RoPE factors
    // After the tensor-core dot products eight threads finish each interleaved row pair, one per peer CTA:
    const int my_pair = tid >> 3;
    const bool pair_live = my_pair < NP;
    const int prow = 2 * (pair_live ? my_pair : 0);  // first local row of the pair
    const bool is_q = prow < QR, is_k = !is_q && prow < QR + KR;
    const int sub = is_q ? prow : (is_k ? prow - QR : prow - QR - KR);
    const int s8 = lane & 7, g4 = lane >> 3;
    const size_t pos_stride = (size_t)kvcols;
    int slot = a.fixed_slot, pos = a.fixed_pos;
    int n_old = 0, chunk = 0, t_begin = 0, t_end = 0;
    const bf16* kb = nullptr;
    const bf16* vb = nullptr;
    uint4 kr[FB_ATT_PRE], vr[FB_ATT_PRE];
    float c0 = 1.f, s0 = 0.f, c1 = 1.f, s1 = 0.f;
    // old keys [0, pos) split over the cluster's CTAs; this CTA's first FB_ATT_PRE blocks are requested
    auto request = [&](int sl, int ps) {
        slot = sl;
        pos = ps;
        n_old = SHORT ? min(pos, 16) : pos;
        chunk = SHORT ? n_old : (n_old + FB_CL - 1) / FB_CL;
        t_begin = SHORT ? 0 : rank * chunk;
        t_end = min(n_old, t_begin + chunk);
        kb = a.k_cache + (size_t)slot * a.max_seq * pos_stride + kvh * HD + s8 * 8;
        vb = a.v_cache + (size_t)slot * a.max_seq * pos_stride + kvh * HD + s8 * 8;
#pragma unroll
        for (int it = 0; it < FB_ATT_PRE; ++it) {
            // SHORT: warp 0 alone takes all (<= 16) keys, four per pass
            const int t = SHORT ? (warp == 0 ? it * 4 + g4 : t_end) : t_begin + it * 32 + warp * 4 + g4;
            if (t < t_end) {
                kr[it] = ldg_stream(kb + (size_t)t * pos_stride);
                vr[it] = ldg_stream(vb + (size_t)t * pos_stride);
            } else {
                kr[it] = make_uint4(0, 0, 0, 0);
                vr[it] = make_uint4(0, 0, 0, 0);
            }
        }
        if (a.rope && (is_q || is_k)) {
            const int dd = (is_q ? rank * QR + sub : rank * KR + sub) & (HD - 1);
            const uint2 f = __ldg(reinterpret_cast<const uint2*>(a.rope + ((size_t)pos * HD + dd) * 2));
            c0 = bf2f(__ushort_as_bfloat16((unsigned short)(f.x & 0xffffu)));
            s0 = bf2f(__ushort_as_bfloat16((unsigned short)(f.x >> 16)));
            c1 = bf2f(__ushort_as_bfloat16((unsigned short)(f.y & 0xffffu)));
            s1 = bf2f(__ushort_as_bfloat16((unsigned short)(f.y >> 16)));
        }
    };
    // A stream's rows before its position were written by earlier frames, so for the backbone they can be requested
    // BEFORE the dependency wait, with the position as it stands in memory now.  It is read again after the wait: if
    // the kernel that sets it had not finished (first layer of a frame), the requests are simply made again.
    bool early = false;
    if constexpr (!SHORT) {
        if (a.row_slot) {
            int sg = __ldcg(a.row_slot), pg = __ldcg(a.row_pos);
            sg = sg < 0 ? 0 : (sg >= a.n_slots ? a.n_slots - 1 : sg);
            pg = pg < 0 ? 0 : (pg >= a.max_seq ? a.max_seq - 1 : pg);
            request(sg, pg);
            early = true;
        }
    }
    pdl_wait();
    fb_stamp(a.dbg, 1);

    int sl = a.fixed_slot, ps = a.fixed_pos;
    if (a.row_slot) {
        sl = __ldcg(a.row_slot);
        ps = __ldcg(a.row_pos);
    }
    float x[EPT];
    load_residual<K, EPT>(a.x_in, a.parts_in, a.n_parts_in, k0, x);
    float nw[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) nw[j] = bf2f(nw_raw[j]);
    if (!early || sl != slot || ps != pos) request(sl, ps);
    fb_stamp(a.dbg, 8);
    if (blockIdx.x == 0) {
        store_bf16<EPT>(a.x_out + k0, x);
        if (a.tap) store_bf16<EPT>(a.tap + k0, x);
    }
    norm_to_smem<K, EPT, FB_WARPS>(x, nw, a.eps, sm.xs, k0, sm.red);
    __syncthreads();
    fb_stamp(a.dbg, 2);
    wait_weights(&sm.bar, a.spin_limit, a.flag);
    cluster_wait();
    fb_stamp(a.dbg, 3);

    // ---- q/k/v rows of this CTA on the tensor cores, results to every CTA of the cluster
    mma_rows<K, S::NR, FB_WARPS>(sm.w, sm.xs, sm.dots, warp, lane);
    __syncthreads();
    if (pair_live) {
        float t0 = rbf(mma_row_total<S::NR, FB_WARPS>(sm.dots, prow));
        float t1 = rbf(mma_row_total<S::NR, FB_WARPS>(sm.dots, prow + 1));
        if (a.rope && (is_q || is_k)) {
            // t*cos + rotate_half(t)*sin, each product and the sum rounded to bf16
            const float o0 = rbf(rbf(t0 * c0) + rbf((-t1) * s0));
            const float o1 = rbf(rbf(t1 * c1) + rbf(t0 * s1));
            t0 = o0;
            t1 = o1;
        }
        // place of the pair inside the head group's [q | k | v] vector; tid & 7 = the peer it goes to
        const int idx = is_q ? rank * QR + sub : (is_k ? G * HD : G * HD + HD) + rank * KR + sub;
        push_f32x2(peer_addr(sm.qkv + idx, tid & 7), peer_addr(&sm.bar_qkv, tid & 7), t0, t1);
        if (!is_q && (tid & 7) == 0) {
            bf16* cache = is_k ? a.k_cache : a.v_cache;
            const int col = kvh * HD + rank * KR + sub;
            *reinterpret_cast<__nv_bfloat162*>(cache + ((size_t)slot * a.max_seq + pos) * pos_stride + col) =
                __floats2bfloat162_rn(t0, t1);
        }
    }
    fb_stamp(a.dbg, 9);
    if (!wait_pushed(&sm.bar_qkv, a.spin_limit) && tid == 0) atomicOr(a.flag, FLAG_COPY_TIMEOUT);
    fb_stamp(a.dbg, 4);

    // ---- attention: this CTA's share of the old keys
    float qf[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        const float4 q0 = *reinterpret_cast<const float4*>(sm.qkv + h * HD + s8 * 8);
        const float4 q1 = *reinterpret_cast<const float4*>(sm.qkv + h * HD + s8 * 8 + 4);
        qf[h][0] = q0.x; qf[h][1] = q0.y; qf[h][2] = q0.z; qf[h][3] = q0.w;
        qf[h][4] = q1.x; qf[h][5] = q1.y; qf[h][6] = q1.z; qf[h][7] = q1.w;
    }
    if constexpr (SHORT) {
        if (warp == 0) {
            // At most 16 old keys and the new one: all scores first, one max, one exponential per key, then the
            // weighted sum - five independent dot products and their butterflies in flight instead of a running
            // (max, sum, accumulator) that every key has to wait for (0.77 -> ~0.4 us per launch, 56 launches a frame).
            float sc[FB_ATT_PRE], vfa[FB_ATT_PRE][8];
#pragma unroll
            for (int it = 0; it < FB_ATT_PRE; ++it) {
                float kf[8];
                unpack8(kr[it], kf);
                unpack8(vr[it], vfa[it]);
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) d = fmaf(qf[0][j], kf[j], d);
                sc[it] = d;
            }
            // the new key (this step's own position) from the exchanged vector
            const float* kn = sm.qkv + G * HD + s8 * 8;
            const float* vn = sm.qkv + G * HD + HD + s8 * 8;
            float dn = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) dn = fmaf(qf[0][j], kn[j], dn);
#pragma unroll
            for (int o = 1; o <= 4; o <<= 1) {
#pragma unroll
                for (int it = 0; it < FB_ATT_PRE; ++it) sc[it] += __shfl_xor_sync(0xffffffffu, sc[it], o);
                dn += __shfl_xor_sync(0xffffffffu, dn, o);
            }
            const float sn = g4 == 0 ? dn * 0.125f : NEG_BIG;   // counted once, by the first key group
            float m = sn;
#pragma unroll
            for (int it = 0; it < FB_ATT_PRE; ++it) {
                sc[it] = it * 4 + g4 < t_end ? sc[it] * 0.125f : NEG_BIG;
                m = fmaxf(m, sc[it]);
            }
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
            const float pn = g4 == 0 ? __expf(sn - m) : 0.f;
            float l = pn, acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = pn * vn[j];
#pragma unroll
            for (int it = 0; it < FB_ATT_PRE; ++it) {
                const float pk = it * 4 + g4 < t_end ? __expf(sc[it] - m) : 0.f;
                l += pk;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(pk, vfa[it][j], acc[j]);
            }
#pragma unroll
            for (int o = 8; o <= 16; o <<= 1) {
                l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
            }
            if (g4 == 0) {
                const float inv = 1.f / l;
#pragma unroll
                for (int j = 0; j < 8; ++j) sm.attn[s8 * 8 + j] = rbf(acc[j] * inv);
            }
        }
        __syncthreads();
        fb_stamp(a.dbg, 12);
    } else {
        if (warp < G) {  // score of the new key (this step's own position), one warp per q head
            const float* q = sm.qkv + warp * HD;
            const float* kn = sm.qkv + G * HD;
            float d = q[lane] * kn[lane] + q[lane + 32] * kn[lane + 32];
            d = warp_sum(d);
            if (lane == 0) sm.s_new[warp] = d * 0.125f;
        }
        float m[G], l[G], acc[G][8];
    #pragma unroll
        for (int h = 0; h < G; ++h) {
            m[h] = NEG_BIG;
            l[h] = 0.f;
    #pragma unroll
            for (int j = 0; j < 8; ++j) acc[h][j] = 0.f;
        }
        auto consume = [&](const uint4& kraw, const uint4& vraw, bool ok) {
            float kf[8], vf[8];
            unpack8(kraw, kf);
            unpack8(vraw, vf);
    #pragma unroll
            for (int h = 0; h < G; ++h) {
                float d = 0.f;
    #pragma unroll
                for (int j = 0; j < 8; ++j) d = fmaf(qf[h][j], kf[j], d);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                if (ok) {
                    const float sc = d * 0.125f;
                    const float mn = fmaxf(m[h], sc);
                    const float corr = __expf(m[h] - mn), p = __expf(sc - mn);
                    l[h] = l[h] * corr + p;
    #pragma unroll
                    for (int j = 0; j < 8; ++j) acc[h][j] = fmaf(p, vf[j], acc[h][j] * corr);
                    m[h] = mn;
                }
            }
        };
    #pragma unroll
        for (int it = 0; it < FB_ATT_PRE; ++it) {
            if (t_begin + it * 32 < t_end) {  // uniform over the CTA
                const int t = t_begin + it * 32 + warp * 4 + g4;
                consume(kr[it], vr[it], t < t_end);
            }
        }
        for (int tb = t_begin + FB_ATT_PRE * 32; tb < t_end; tb += 32) {  // longer caches: the rest, block by block
            const int t = tb + warp * 4 + g4;
            const bool ok = t < t_end;
            const uint4 kraw = ok ? ldg_stream(kb + (size_t)t * pos_stride) : make_uint4(0, 0, 0, 0);
            const uint4 vraw = ok ? ldg_stream(vb + (size_t)t * pos_stride) : make_uint4(0, 0, 0, 0);
            consume(kraw, vraw, ok);
        }
        // merge the warp's 4 key groups, then the CTA's 8 warps
    #pragma unroll
        for (int o = 8; o <= 16; o <<= 1) {
    #pragma unroll
            for (int h = 0; h < G; ++h) {
                const float mo = __shfl_xor_sync(0xffffffffu, m[h], o);
                const float lo = __shfl_xor_sync(0xffffffffu, l[h], o);
                float ao[8];
    #pragma unroll
                for (int j = 0; j < 8; ++j) ao[j] = __shfl_xor_sync(0xffffffffu, acc[h][j], o);
                softmax_merge(m[h], l[h], acc[h], mo, lo, ao);
            }
        }
        if (g4 == 0) {
    #pragma unroll
            for (int h = 0; h < G; ++h) {
    #pragma unroll
                for (int j = 0; j < 8; ++j) sm.wpart[warp][h][s8][j] = acc[h][j];
                sm.wpart[warp][h][s8][8] = m[h];
                sm.wpart[warp][h][s8][9] = l[h];
            }
        }
        __syncthreads();
        fb_stamp(a.dbg, 10);
        const int th = tid >> 6, tdim = tid & 63;  // thread (q head, dim) for tid < G * 64
        if (tid < G * HD) {
            const int ds = tdim >> 3, dj = tdim & 7;
            float M_ = NEG_BIG;
    #pragma unroll
            for (int w = 0; w < FB_WARPS; ++w) M_ = fmaxf(M_, sm.wpart[w][th][ds][8]);
            float L_ = 0.f, O_ = 0.f;
    #pragma unroll
            for (int w = 0; w < FB_WARPS; ++w) {
                const float c = __expf(sm.wpart[w][th][ds][8] - M_);
                L_ += sm.wpart[w][th][ds][9] * c;
                O_ += sm.wpart[w][th][ds][dj] * c;
            }
    #pragma unroll
            for (int c = 0; c < FB_CL; ++c) {
                float* mine = &sm.part[0][0][0] + (rank * G + th) * (HD + 2);
                const uint32_t pbar = peer_addr(&sm.bar_part, c);
                push_f32(peer_addr(mine + tdim, c), pbar, O_);
                if (tdim == 0) push_f32x2(peer_addr(mine + HD, c), pbar, M_, L_);
            }
        }
        __syncthreads();
        fb_stamp(a.dbg, 11);
        if (!wait_pushed(&sm.bar_part, a.spin_limit) && tid == 0) atomicOr(a.flag, FLAG_COPY_TIMEOUT);
        fb_stamp(a.dbg, 5);
        if (tid < G * HD) {
            // every CTA merges the partial states in CTA order, then the new key: same bits everywhere
            float Mx = sm.s_new[th];
    #pragma unroll
            for (int c = 0; c < FB_CL; ++c) Mx = fmaxf(Mx, sm.part[c][th][HD]);
            float Ls = 0.f, Os = 0.f;
    #pragma unroll
            for (int c = 0; c < FB_CL; ++c) {
                const float e = __expf(sm.part[c][th][HD] - Mx);
                Ls += sm.part[c][th][HD + 1] * e;
                Os += sm.part[c][th][tdim] * e;
            }
            const float en = __expf(sm.s_new[th] - Mx);
            Ls += en;
            Os += en * sm.qkv[G * HD + HD + tdim];
            sm.attn[th * HD + tdim] = rbf(Os / Ls);
        }
        __syncthreads();
        fb_stamp(a.dbg, 12);

    }

    // ---- this head group's K-slice of out_proj for the CTA's rows
    small_matvec<OC, OR / FB_WARPS>(sm.wo, sm.attn, warp * (OR / FB_WARPS), a.parts_out + (size_t)kvh * K + rank * OR, lane);
    fb_stamp(a.dbg, 6);
}

// ---------------------------------------------------------------------------
// MLP block
// ---------------------------------------------------------------------------
struct MlpBlockArgs {
    const bf16* x_in;       // (K) x as the attention block saw it
    const float* parts_in;  // (n_parts_in, K) out_proj partial rows
    int n_parts_in;
    bf16* x_out;            // (K) x after the attention residual (read by the next attention block)
    const bf16* norm_w;
    float eps;
    const bf16* w1;         // (F, K)
    const bf16* w3;         // (F, K)
    const bf16* w2;         // (K, F)
    float* parts_out;       // (clusters, K)
    // optional: warm L2 with the K/V rows the next attention block reads (rows before the row's position
    // do not change during a frame)
    const bf16* next_k;
    const bf16* next_v;
    const int32_t* row_slot;
    const int32_t* row_pos;
    int max_seq, kvcols, n_slots;
    int32_t* flag;
    unsigned spin_limit;
    PrefetchList next;
    unsigned long long* dbg;
};

// U hidden units per CTA; the grid is F / (U * FB_CL) clusters.
template <int K, int F, int U, int TH>
struct MlpBlockSmem {
    static constexpr int CU = U * FB_CL;     // hidden units of the cluster
    static constexpr int OR = K / FB_CL;     // w2 rows of this CTA
    static constexpr int NCL = F / CU;       // clusters
    static_assert(F % CU == 0 && CU % 8 == 0, "ffn must split evenly into 16-byte pieces");
    alignas(128) bf16 w2[OR * CU];           // destination of a tiled copy: first, 128-byte aligned
    alignas(16) bf16 w13[2 * U * K];         // w1 rows of this CTA's units, then their w3 rows
    alignas(16) bf16 xs[K];
    alignas(16) float g[CU];
    float red[TH / 32];
    float dots[(TH / 32) * ((2 * U + 15) / 16) * 16];  // per-warp partial sums of the w1 / w3 rows
    alignas(8) uint64_t bar;     // weight copies
    alignas(8) uint64_t bar_g;   // the cluster's activations complete (all peers' units)
    alignas(8) uint64_t bar_w2;  // the w2 slice, when it is copied after the dependency wait
};

template <int K, int F, int U, int TH>
__global__ void __launch_bounds__(TH, 1) k_mlp_block(const __grid_constant__ CUtensorMap map_w2, MlpBlockArgs a) {
    using S = MlpBlockSmem<K, F, U, TH>;
    constexpr int EPT = K / TH;
    constexpr int NWARP = TH / 32;
    constexpr int CU = S::CU, OR = S::OR;
    // The backbone's w2 slice (6 MB over the grid, needed last) is copied only once this kernel's residual is in: before
    // that it would travel together with the attention block's own loads, which are on the chain (0.794 -> 0.786 ms).
    // The depth block's slice is small and its chain tighter: there the late copy cost 0.005 ms.
    constexpr bool LATE_W2 = K >= 1024;
    extern __shared__ __align__(128) unsigned char fb_smem[];
    S& sm = *reinterpret_cast<S*>(fb_smem);
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int cid = blockIdx.x / FB_CL;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    fb_stamp(a.dbg, 0);
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            mbar_init(&sm.bar, 1);
            mbar_init(&sm.bar_g, 1);
            mbar_init(&sm.bar_w2, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&sm.bar_g, (uint32_t)(CU * 4));
        }
    }
    __syncthreads();
    cluster_arrive_relaxed();  // after the mbarriers exist, before the weight copies are issued (see the attention block)
    if (tid == 0) {
        mbar_expect_tx(&sm.bar, (uint32_t)(2 * U * K * 2 + (LATE_W2 ? 0 : OR * CU * 2)));
        const size_t u0 = (size_t)cid * CU + rank * U;
        bulk_g2s(sm.w13, a.w1 + u0 * K, U * K * 2, &sm.bar);
        bulk_g2s(sm.w13 + U * K, a.w3 + u0 * K, U * K * 2, &sm.bar);
        // the w2 slice (OR rows x CU columns) as ONE tiled copy
        if constexpr (!LATE_W2) tma_load_2d(sm.w2, &map_w2, cid * CU, rank * OR, &sm.bar);
    }
    if (cid < FB_HINT_CLUSTERS) prefetch_l2(a.next, TH);   // a hint: partial coverage is fine
    const int k0 = tid * EPT;
    // Requested here, converted after the wait: the clusters of this kernel that only become resident when the
    // attention block's CTAs leave (at most 15 clusters of 8 fit the part at once) run this prologue ON the chain,
    // so nothing in it may wait for a load.
    alignas(8) bf16 nw_raw[EPT];
    if constexpr (EPT == 4) *reinterpret_cast<uint2*>(nw_raw) = __ldg(reinterpret_cast<const uint2*>(a.norm_w + k0));
    else *reinterpret_cast<unsigned*>(nw_raw) = __ldg(reinterpret_cast<const unsigned*>(a.norm_w + k0));
    if (a.next_k && cid < FB_HINT_CLUSTERS) {   // the hints are the early clusters' job, for the same reason
        // The next layer's K/V rows are asked into L2 BEFORE the dependency wait (after it, the dependent load of the
        // position and the address arithmetic sat on the chain to the norm: 0.6 us per layer).  The rows before the
        // stream's position do not change during a frame.  The position itself may still be last frame's here (the
        // kernel that writes it need not have finished): then one row is not asked for, nothing more - these are
        // hints, and slot and position are clamped so that every address lies inside the cache.
        int slot = __ldcg(a.row_slot), pos = __ldcg(a.row_pos);
        slot = slot < 0 ? 0 : (slot >= a.n_slots ? a.n_slots - 1 : slot);
        pos = pos < 0 ? 0 : (pos > a.max_seq ? a.max_seq : pos);
        const size_t row_bytes = (size_t)a.kvcols * sizeof(bf16);
        const size_t lines = (size_t)pos * row_bytes / 128;
        const char* kbase = reinterpret_cast<const char*>(a.next_k) + (size_t)slot * a.max_seq * row_bytes;
        const char* vbase = reinterpret_cast<const char*>(a.next_v) + (size_t)slot * a.max_seq * row_bytes;
        const size_t n_hint = (size_t)(gridDim.x < FB_HINT_CLUSTERS * FB_CL ? gridDim.x : FB_HINT_CLUSTERS * FB_CL) * TH;
        for (size_t i = (size_t)blockIdx.x * TH + tid; i < 2 * lines; i += n_hint) {
            const char* p = i < lines ? kbase + i * 128 : vbase + (i - lines) * 128;   // one 128-byte line each
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
        }
    }
    pdl_wait();
    fb_stamp(a.dbg, 1);

    float x[EPT];
    load_residual<K, EPT>(a.x_in, a.parts_in, a.n_parts_in, k0, x);
    float nw[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) nw[j] = bf2f(nw_raw[j]);
    if (blockIdx.x == 0) store_bf16<EPT>(a.x_out + k0, x);
    norm_to_smem<K, EPT, NWARP>(x, nw, a.eps, sm.xs, k0, sm.red);
    __syncthreads();
    fb_stamp(a.dbg, 2);
    if (LATE_W2 && tid == 0) {   // needed last: requested once the residual is in
        mbar_expect_tx(&sm.bar_w2, (uint32_t)(OR * CU * 2));
        tma_load_2d(sm.w2, &map_w2, cid * CU, rank * OR, &sm.bar_w2);
    }
    wait_weights(&sm.bar, a.spin_limit, a.flag);
    cluster_wait();
    fb_stamp(a.dbg, 3);

    // ---- SiLU(w1 h) * (w3 h) for this CTA's hidden units: rows on the tensor cores, then eight threads
    //      per unit, one per peer CTA
    static_assert(U * FB_CL <= TH, "eight threads finish each hidden unit");
    mma_rows<K, 2 * U, NWARP>(sm.w13, sm.xs, sm.dots, warp, lane);
    __syncthreads();
    if (tid < U * FB_CL) {
        const int u = tid >> 3;
        const float a1 = rbf(mma_row_total<2 * U, NWARP>(sm.dots, u));
        const float a3 = rbf(mma_row_total<2 * U, NWARP>(sm.dots, U + u));
        const float sl = rbf(a1 / (1.0f + expf(-a1)));
        push_f32(peer_addr(sm.g + rank * U + u, tid & 7), peer_addr(&sm.bar_g, tid & 7), rbf(sl * a3));
    }
    fb_stamp(a.dbg, 9);
    if (!wait_pushed(&sm.bar_g, a.spin_limit) && tid == 0) atomicOr(a.flag, FLAG_COPY_TIMEOUT);
    fb_stamp(a.dbg, 4);

    // ---- the cluster's K-slice of w2 for this CTA's rows
    static_assert(OR % NWARP == 0, "rows split evenly over the warps");
    if constexpr (LATE_W2) wait_weights(&sm.bar_w2, a.spin_limit, a.flag);
    small_matvec<CU, OR / NWARP>(sm.w2, sm.g, warp * (OR / NWARP), a.parts_out + (size_t)cid * K + rank * OR, lane);
    fb_stamp(a.dbg, 6);
}

}  // namespace vuib
