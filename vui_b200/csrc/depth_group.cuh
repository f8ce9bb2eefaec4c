// The depth transformer's whole codebook loop for MANY streams in one launch.
//
// With 5+ streams per step the per-launch path runs ~420 small tensor-core GEMM launches per frame
// for the depth loop (15 codebooks x 4 layers x 7 kernels), each a chain of fixed latencies.  Here a
// thread-block cluster of 8 CTAs owns a GROUP of R streams for the whole loop: nothing crosses
// clusters, so there is no kernel hand-over inside the loop at all.  The depth weights (25.7 MB + one
// 2 MB head per codebook) stay resident in L2 and every cluster streams them through a ring of
// shared-memory boxes; that is redundant L2 traffic (clusters x 27.7 MB per codebook), which the L2
// has to spare, in exchange for ~400 hand-overs.
//
//  * CTA c of a cluster is attention head c, hidden-unit slice c of the MLP and row slice c of each head
//    matrix.  Per layer: RMSNorm (replicated) -> its head's q/k/v rows -> its head's attention over its
//    own K/V (global scratch only this CTA touches) -> its K-slice of out_proj for ALL output rows ->
//    reduce-scatter of the partial rows over the cluster (st.async pushes into the owner's landing
//    zone, summed in source order) -> residual add -> all-gather of the new residual slice; the same
//    for w1/w3 -> SiLU*gate -> its K-slice of w2.
//  * Weights arrive as 64 x 64 bf16 boxes (128-byte swizzle) through TMA from a dedicated producer warp
//    that runs ahead through the whole schedule (layers, positions, heads), so the stream never stops
//    at a phase boundary; 8 consumer warps run mma.sync m16n8k16 (weights = M side via ldmatrix, the R
//    streams = N side), warps 0-3 on the even boxes of a row group, warps 4-7 on the odd ones.
//  * After a position's layers the 8 CTAs write their logits slices, signal each other through
//    mbarriers, and CTA n samples stream n with the per-launch path's sampler (same Philox keys, same
//    draws), building the next position's token.
//
// Measured: a cluster streams its boxes at ~45 GB/s per SM (~360 GB/s for the 8 SMs, which share one
// GPC's path to the L2) whether 1 or 8 clusters run and whether or not the boxes are read, so the loop
// costs ~2.0 ms per frame for any stream count up to 120 (groups of 8) - the per-launch path takes
// 2.95 ms at 64 streams - and breaks even with it at 256 streams (groups of 16, two waves).
//
// Rounding points are those of the per-launch path (src/vui/model.py:577-635, 908-986); sums are
// fp32 in another order.  Every wait is bounded; a CTA whose wait runs out records the device flag
// and skips the rest of its waits.  No TMA load uses cluster multicast.
#pragma once
#include "fused_blocks.cuh"

namespace vuib {

constexpr int DG_CL = 8;
constexpr int DG_CONSUMERS = 256;
constexpr int DG_THREADS = DG_CONSUMERS + 128;   // two consumer warpgroups + one whose first warp is the producer
constexpr int DG_RING = 16;          // boxes in the ring
constexpr int DG_STAGE = 4;          // boxes per stage: one full / empty mbarrier pair, one producer wake-up
constexpr int DG_STAGES = DG_RING / DG_STAGE;
static_assert(DG_STAGE == 4 && DG_RING == 16, "dg_rowgroup shifts by these");
constexpr int DG_BOX_BYTES = 64 * 64 * 2;
constexpr int DG_LAYERS = 4;
constexpr int DG_D = 512;
constexpr int DG_XS = DG_D + 8;   // padded row strides (elements): conflict-free B-fragment loads
constexpr int DG_GS = 192 + 8;
constexpr int DG_AS = HD + 8;

// The weights reach the ring as ONE contiguous 32 KB bulk copy per stage (four boxes): measured on this part, a
// tiled TMA box (64 rows of 128 bytes, 1-2.8 KB apart in the matrix) arrives at ~43 GB/s per SM however many are
// in flight or however many lanes request them, a contiguous 32 KB bulk copy at ~200 GB/s.  So the depth weights
// are copied once, when they are bound, into a "box stream": for every (layer, CTA of the cluster) the boxes in
// exactly the order the kernel consumes them, each box already in its 128-byte-swizzled shared-memory image
// (row r, 16-byte piece q at r * 128 + ((q ^ (r & 7)) << 4)); the heads of the 15 codebooks likewise per
// (codebook, CTA).  Rows or columns beyond a matrix are zeros, as the tensor-map fill was.
struct DepthGroupStream {
    const unsigned char* layers;   // [n_layers][8 CTAs][boxes_per_layer][8192]
    const unsigned char* head;     // [Q - 1][8 CTAs][32][8192]
    int boxes_per_layer;           // 32 + 24 * n_ub
};

__host__ __device__ inline int dg_boxes_per_layer(int n_ub) { return 24 + 8 + 16 * n_ub + 8 * n_ub; }

struct DgStreamBuild {
    const bf16* wqkv[DG_LAYERS]; const bf16* out[DG_LAYERS]; const bf16* w1[DG_LAYERS]; const bf16* w3[DG_LAYERS];
    const bf16* w2[DG_LAYERS];
    const bf16* head;              // ((Q - 1) * CS, 512)
    unsigned char* layers; unsigned char* head_out;
    int n_layers, ffn, upc, n_ub, CS, n_head_pos;   // n_head_pos = Q - 1
};

// One CTA per box of the stream; the box sequence of a layer is q|k|v rows of head c (8 K-chunks each), the
// head's K-slice of out_proj (8 row blocks), w1/w3 of the CTA's hidden units (per 64 units: the 8 K-chunks of w1, then
// the 8 of w3), the CTA's K-slice of w2 (8 row blocks x n_ub column blocks).
__global__ void __launch_bounds__(256) k_build_dg_stream(DgStreamBuild b) {
    const int bpl = dg_boxes_per_layer(b.n_ub);
    const int n_layer_boxes = b.n_layers * DG_CL * bpl;
    int box = blockIdx.x;
    const bf16* W;
    int N, K, x, y;
    unsigned char* dst;
    if (box < n_layer_boxes) {
        const int l = box / (DG_CL * bpl), c = (box / bpl) % DG_CL;
        int j = box % bpl;
        dst = b.layers + (size_t)box * DG_BOX_BYTES;
        if (j < 24) { W = b.wqkv[l]; N = 3 * DG_D; K = DG_D; x = (j % 8) * 64; y = (j / 8) * DG_D + c * HD; }
        else if ((j -= 24) < 8) { W = b.out[l]; N = DG_D; K = DG_D; x = c * HD; y = j * 64; }
        else if ((j -= 8) < 16 * b.n_ub) {
            const int ub = j / 16, kb = j % 8;
            W = (j % 16) >= 8 ? b.w3[l] : b.w1[l]; N = b.ffn; K = DG_D; x = kb * 64; y = c * b.upc + ub * 64;
        } else {
            j -= 16 * b.n_ub;
            W = b.w2[l]; N = DG_D; K = b.ffn; x = c * b.upc + (j % b.n_ub) * 64; y = (j / b.n_ub) * 64;
        }
    } else {
        box -= n_layer_boxes;
        const int p = box / (DG_CL * 32), c = (box / 32) % DG_CL, j = box % 32;
        dst = b.head_out + (size_t)box * DG_BOX_BYTES;
        W = b.head; N = b.n_head_pos * b.CS; K = DG_D; x = (j % 8) * 64; y = p * b.CS + c * 256 + (j / 8) * 64;
    }
    for (int i = threadIdx.x; i < 64 * 8; i += 256) {       // 16-byte pieces: row r, piece q
        const int r = i >> 3, q = i & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (y + r < N) {
            const int col = x + q * 8;
            if (col + 8 <= K) v = __ldg(reinterpret_cast<const uint4*>(W + (size_t)(y + r) * K + col));
            else if (col < K) {
                bf16 tmp[8];
                for (int e = 0; e < 8; ++e) tmp[e] = col + e < K ? W[(size_t)(y + r) * K + col + e] : f2bf(0.f);
                v = *reinterpret_cast<const uint4*>(tmp);
            }
        }
        *reinterpret_cast<uint4*>(dst + r * 128 + ((q ^ (r & 7)) << 4)) = v;
    }
}

struct DepthGroupArgs {
    int B;            // streams
    int n_layers;     // <= DG_LAYERS
    int Q, Qn;        // quantizers of the model, codebooks to emit (positions to run)
    int CS;
    int upc;          // hidden units per CTA = rq_ffn / 8 (<= 192)
    int max_rows;     // row stride of the depth K/V scratch
    float eps;
    const bf16* x2;   // (B, 2, 512): tokens of depth positions 0 and 1
    bf16* x1;         // (B, 512): token of the next position, written by the sampler
    bf16* kc;         // (layers, max_rows, Q, 512)
    bf16* vc;
    const bf16* attn_norm[DG_LAYERS];
    const bf16* mlp_norm[DG_LAYERS];
    const bf16* final_norm;
    bf16* logits;     // (B, CS) scratch
    bf16* tap;        // optional copy of the logits: row stride (Q-1)*CS, codebook i at +i*CS
    SampleArgs sa;    // everything but the per-position fields
    int32_t* flag;
    unsigned spin_limit;
    unsigned long long* dbg;  // optional: device-clock stamps of CTA 0 at position 8, layer 1 (profiling aid)
};

template <int R>
struct DepthGroupSmem {
    static constexpr int NT = R / 8;
    alignas(1024) unsigned char ring[DG_RING][DG_BOX_BYTES];
    alignas(16) bf16 x[R][DG_XS];        // residual stream of the group's streams (same in every CTA)
    alignas(16) bf16 h[R][DG_XS];        // normed activations
    alignas(16) bf16 attn[R][DG_AS];     // this head's attention output
    alignas(16) bf16 g[R][DG_GS];        // this CTA's SwiGLU activations (zero past its units)
    alignas(16) float q[R][HD];          // this head's q, new k, new v (bf16 values)
    alignas(16) float kn[R][HD];
    alignas(16) float vn[R][HD];
    alignas(16) float land[DG_CL][R][HD];  // reduce-scatter landing zone [source CTA][stream][column]
    alignas(16) float comb[2][4][32][NT * 4];  // accumulators of warps 4-7 handed to warps 0-3 (double-buffered)
    alignas(8) uint64_t full[DG_STAGES];
    alignas(8) uint64_t empty[DG_STAGES];
    alignas(8) uint64_t bar_rs, bar_ag, bar_logits, bar_x;
    SampleSmem samp;
};

__device__ __forceinline__ void dg_bar() { bar_named(1, DG_CONSUMERS); }

__device__ __forceinline__ void remote_arrive(const uint64_t* local_bar, int peer) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_addr(local_bar, peer)) : "memory");
}

// Bounded wait with cluster-scope acquire on one phase parity.
__device__ __forceinline__ bool dg_wait(uint64_t* bar, unsigned parity, unsigned limit) {
    const uint32_t a = smem_u32(bar);
    for (unsigned spins = 0; spins < limit; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void push_b32(uint32_t dst, uint32_t bar, uint32_t v) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(dst), "r"(v), "r"(bar) : "memory");
}

// Consumer-side state every helper below shares (identical in all 256 consumer threads except `dead`).
struct DgState {
    int bi;         // boxes of the schedule passed so far
    int comb_buf;   // which hand-over buffer the next combine() uses
    bool dead;      // a wait of this thread ran out: skip the rest of its waits
    int waited;     // the stage fill (bi / DG_STAGE) this thread last waited for: its other boxes need no second wait
    int32_t* flag;
    unsigned limit;
};

// Wait on a barrier that only this CTA's own copies complete (the weight ring): CTA scope is enough.
__device__ __forceinline__ void dg_wait_local_or_die(DgState& st, uint64_t* bar, unsigned parity) {
    if (st.dead) return;
    if (!mbar_wait(bar, parity, st.limit)) {
        if ((threadIdx.x & 31) == 0) atomicOr(st.flag, FLAG_COPY_TIMEOUT);
        st.dead = true;
    }
}

__device__ __forceinline__ void dg_wait_or_die(DgState& st, uint64_t* bar, unsigned parity) {
    if (st.dead) return;
    if (!dg_wait(bar, parity, st.limit)) {
        if ((threadIdx.x & 31) == 0) atomicOr(st.flag, FLAG_COPY_TIMEOUT);
        st.dead = true;
    }
}

// One row group of 64 weight rows: `nbox` boxes; its slice of the activation rows starts at element
// (j >> kshift) * kmul.  owner < 0: box j is read by warp set (j & 1) and the two sets' sums are combined
// afterwards (dg_combine); owner = 0 / 1: that set reads every box and owns the result, the other set skips the
// row group - successive row groups then alternate between the sets and need neither a combine nor a barrier.
// Leaves this warp's accumulators in acc.
template <int R>
__device__ __forceinline__ void dg_rowgroup(DepthGroupSmem<R>& sm, DgState& st, int nbox, const bf16* act, int astride,
                                            int kshift, int kmul, float (&acc)[R / 8][4], int owner = -1) {
    constexpr int NT = R / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int set = warp >> 2, mt = warp & 3;
    const int base = st.bi;
    st.bi += nbox;
    // A warp runs this loop alone on its scheduler, so every dependent instruction of the per-box bookkeeping costs
    // its full latency: a box is ~60 instructions here (it was ~300 with per-element activation loads and 64-bit
    // address arithmetic, 490 cycles per box against the 128 the shared-memory port allows).  Everything that does
    // not change from box to box is computed once: the lane's four ldmatrix offsets into a swizzled box, and the
    // lane's row address for the activation fragments, which are ldmatrix loads too (an activation row is k-major,
    // so a non-transposed 8x8 matrix is the B fragment of eight streams).
    // The four k-steps of a box go to four independent accumulators (added at the end), and the fragments of the
    // warp's next box are fetched while the MMAs of the current one are in flight.
    float c4[4][NT][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) c4[ks][nt][0] = c4[ks][nt][1] = c4[ks][nt][2] = c4[ks][nt][3] = 0.f;
    struct Frag { uint32_t a[4][4]; uint32_t b[4][NT][2]; };
    Frag f0, f1;   // two named buffers (a run-time buffer index would put them in local memory)
    const int first = owner < 0 ? set : 0, step = owner < 0 ? 2 : 1;   // this set's boxes: first, first + step, ...
    const bool mine = owner < 0 || owner == set;
    uint32_t a_off[4];
    {
        const int row = mt * 16 + (lane & 15);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) a_off[ks] = (uint32_t)(row * 128 + (((ks * 2 + (lane >> 4)) ^ (row & 7)) << 4));
    }
    const uint32_t ring_s = smem_u32(sm.ring[0]), empty_s = smem_u32(&sm.empty[0]);
    // matrix (lane >> 3) of an x4 load is k-offset 8 * (lane >> 3); its row (lane & 7) is stream nt * 8 + (lane & 7)
    const uint32_t b_row = smem_u32(act) + (uint32_t)(((lane & 7) * astride + (lane >> 3) * 8) * 2);
    auto fetch = [&](int j, Frag& f) {
        const int bi = base + j;
        if ((bi >> 2) != st.waited) {   // an mbarrier wait costs ~250 cycles even when the copy has landed
            dg_wait_local_or_die(st, &sm.full[(bi & (DG_RING - 1)) >> 2], (bi / DG_RING) & 1);
            st.waited = bi >> 2;
        }
        const uint32_t bx = ring_s + (uint32_t)((bi & (DG_RING - 1)) * DG_BOX_BYTES);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(f.a[ks][0]), "=r"(f.a[ks][1]), "=r"(f.a[ks][2]), "=r"(f.a[ks][3])
                         : "r"(bx + a_off[ks]));
        const uint32_t kb = b_row + (uint32_t)(((j >> kshift) * kmul) * 2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t ba = kb + (uint32_t)(nt * 8 * astride * 2);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(f.b[0][nt][0]), "=r"(f.b[0][nt][1]), "=r"(f.b[1][nt][0]), "=r"(f.b[1][nt][1])
                         : "r"(ba));
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(f.b[2][nt][0]), "=r"(f.b[2][nt][1]), "=r"(f.b[3][nt][0]), "=r"(f.b[3][nt][1])
                         : "r"(ba + 64));
        }
    };
    // MMAs of box j, then its release: issuing the MMAs has taken the box's fragments out of shared memory
    auto consume = [&](int j, const Frag& f) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(c4[ks][nt][0]), "+f"(c4[ks][nt][1]), "+f"(c4[ks][nt][2]), "+f"(c4[ks][nt][3])
                             : "r"(f.a[ks][0]), "r"(f.a[ks][1]), "r"(f.a[ks][2]), "r"(f.a[ks][3]),
                               "r"(f.b[ks][nt][0]), "r"(f.b[ks][nt][1]));
        __syncwarp();
        if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];"
                         ::"r"(empty_s + (uint32_t)((((base + j) & (DG_RING - 1)) >> 2) * 8)) : "memory");
    };
    if (mine) {
        if (first < nbox) fetch(first, f0);
#pragma unroll
        for (int j = first; j < nbox; j += 2 * step) {
            if (j + step < nbox) fetch(j + step, f1);      // requested before the MMAs of box j are issued
            consume(j, f0);
            if (j + step < nbox) {
                if (j + 2 * step < nbox) fetch(j + 2 * step, f0);
                consume(j + step, f1);
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = (c4[0][nt][i] + c4[1][nt][i]) + (c4[2][nt][i] + c4[3][nt][i]);
}

// Hand the odd-box accumulators (warps 4-7) to the even-box warps (0-3); true in the warps that go on
// with the row group's epilogue, `other` holding the partner's values.
template <int R>
__device__ __forceinline__ bool dg_combine(DepthGroupSmem<R>& sm, DgState& st, const float (&acc)[R / 8][4],
                                           float (&other)[R / 8][4]) {
    constexpr int NT = R / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int set = warp >> 2, mt = warp & 3;
    float* cb = &sm.comb[st.comb_buf][mt][lane][0];
    if (set == 1) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) cb[nt * 4 + i] = acc[nt][i];
    }
    dg_bar();
    if (set == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) other[nt][i] = cb[nt * 4 + i];
    }
    st.comb_buf ^= 1;
    return set == 0;
}

// RMSNorm of the residual rows into sm.h: warp w takes streams w, w + 8, ...
template <int R>
__device__ __forceinline__ void dg_norm(DepthGroupSmem<R>& sm, const bf16* w, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float wf[16];
    {
        float t0[8], t1[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(w + lane * 16)), t0);
        unpack8(__ldg(reinterpret_cast<const uint4*>(w + lane * 16 + 8)), t1);
#pragma unroll
        for (int j = 0; j < 8; ++j) { wf[j] = t0[j]; wf[8 + j] = t1[j]; }
    }
    for (int n = warp; n < R; n += DG_CONSUMERS / 32) {
        float v[16], t0[8], t1[8];
        unpack8(*reinterpret_cast<const uint4*>(&sm.x[n][lane * 16]), t0);
        unpack8(*reinterpret_cast<const uint4*>(&sm.x[n][lane * 16 + 8]), t1);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j] = t0[j]; v[8 + j] = t1[j]; }
#pragma unroll
        for (int j = 0; j < 16; ++j) ss = fmaf(v[j], v[j], ss);
        ss = warp_sum(ss);
        const float rinv = rsqrtf(ss / (float)DG_D + eps);
        float o0[8], o1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { o0[j] = rbf(v[j] * rinv) * wf[j]; o1[j] = rbf(v[8 + j] * rinv) * wf[8 + j]; }
        *reinterpret_cast<uint4*>(&sm.h[n][lane * 16]) = pack8(o0);
        *reinterpret_cast<uint4*>(&sm.h[n][lane * 16 + 8]) = pack8(o1);
    }
}

// Partial rows of a column-split product go to the CTA that owns those 64 output columns.
template <int R>
__device__ __forceinline__ void dg_push_partial(DepthGroupSmem<R>& sm, int c, int rb, const float (&acc)[R / 8][4]) {
    constexpr int NT = R / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = warp & 3, g = lane >> 2, t = lane & 3;
    const uint32_t pbar = peer_addr(&sm.bar_rs, rb);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = nt * 8 + 2 * t + (i & 1), col = mt * 16 + g + (i >> 1) * 8;
            push_f32(peer_addr(&sm.land[c][n][col], rb), pbar, acc[nt][i]);
        }
}

// Once all eight sources have landed, the owner adds them in source order to the residual and sends
// the new slice to every CTA's copy of x.
template <int R>
__device__ __forceinline__ void dg_residual_exchange(DepthGroupSmem<R>& sm, DgState& st, int c, unsigned& ph_rs,
                                                     unsigned& ph_ag) {
    const int tid = threadIdx.x;
    dg_wait_or_die(st, &sm.bar_rs, ph_rs & 1);
    ++ph_rs;
    if (tid == 0) mbar_expect_tx(&sm.bar_rs, (uint32_t)(DG_CL * R * HD * 4));  // armed for the next round
    for (int e = tid; e < R * (HD / 2); e += DG_CONSUMERS) {
        const int n = e / (HD / 2), cp = (e % (HD / 2)) * 2;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int src = 0; src < DG_CL; ++src) {
            s0 += sm.land[src][n][cp];
            s1 += sm.land[src][n][cp + 1];
        }
        const __nv_bfloat162 xo = *reinterpret_cast<const __nv_bfloat162*>(&sm.x[n][c * HD + cp]);
        const __nv_bfloat162 xn = __floats2bfloat162_rn(__low2float(xo) + rbf(s0), __high2float(xo) + rbf(s1));
        const uint32_t bits = *reinterpret_cast<const uint32_t*>(&xn);
#pragma unroll
        for (int p = 0; p < DG_CL; ++p) push_b32(peer_addr(&sm.x[n][c * HD + cp], p), peer_addr(&sm.bar_ag, p), bits);
    }
    dg_wait_or_die(st, &sm.bar_ag, ph_ag & 1);
    ++ph_ag;
    if (tid == 0) mbar_expect_tx(&sm.bar_ag, (uint32_t)(DG_CL * R * HD * 2));
    dg_bar();
}

template <int R>
__global__ void __launch_bounds__(DG_THREADS, 1)
k_depth_group(const DepthGroupStream strm, DepthGroupArgs a) {
    using S = DepthGroupSmem<R>;
    constexpr int NT = S::NT;
    extern __shared__ __align__(1024) unsigned char dg_smem[];
    S& sm = *reinterpret_cast<S*>(dg_smem);
    cg::cluster_group cluster = cg::this_cluster();
    const int c = (int)cluster.block_rank();           // head / slice of this CTA
    const int b0 = (blockIdx.x / DG_CL) * R;           // first stream of the group
    const int n_valid = min(R, a.B - b0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();

    if (tid == 0) {
        for (int i = 0; i < DG_STAGES; ++i) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], 4 * DG_STAGE);  // every box of the stage is read by four warps
        }
        mbar_init(&sm.bar_rs, 1);
        mbar_init(&sm.bar_ag, 1);
        mbar_init(&sm.bar_logits, DG_CL);
        mbar_init(&sm.bar_x, DG_CL);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(&sm.bar_rs, (uint32_t)(DG_CL * R * HD * 4));
        mbar_expect_tx(&sm.bar_ag, (uint32_t)(DG_CL * R * HD * 2));
    }
    __syncthreads();
    cluster_arrive();

    const int n_pos = a.Qn;  // depth positions 0 .. Qn-1; position p >= 1 yields codebook p
    const int n_ub = (a.upc + 63) / 64;

    // Registers: a CTA of 384 threads starts with 168 per thread.  The producer's warpgroup gives most of its
    // share back and the two consumer warpgroups take it (setmaxnreg is a warpgroup-wide instruction: all four
    // warps of each group execute it), so the consumers can hold a second set of fragments in flight.
    // (The two paths never meet again: the compiler allocates registers for each under its own limit.)
    // ------------------------------------------------------------------ producer warpgroup
    if (warp >= DG_CONSUMERS / 32) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
        if (warp > DG_CONSUMERS / 32) {   // the producer's three idle companions
            cluster_wait();
            return;
        }
        if (lane == 0) {
            int i = 0;   // stages issued so far (a stage = DG_STAGE consecutive boxes = one contiguous 32 KB copy)
            bool dead = false;
            // A stage is re-armed once its previous boxes have all been read; the wait polls without suspending, so
            // that the producer wakes as soon as the last reader arrives.
            auto issue_stage = [&](const unsigned char* src) {
                if (dead) return;
                const int stage = i % DG_STAGES;
                if (i >= DG_STAGES) {
                    const uint32_t ea = smem_u32(&sm.empty[stage]);
                    const unsigned parity = ((i / DG_STAGES) - 1) & 1;
                    unsigned spins = 0;
                    for (;;) {
                        uint32_t ok;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                            "selp.u32 %0, 1, 0, p;\n\t}"
                            : "=r"(ok)
                            : "r"(ea), "r"(parity)
                            : "memory");
                        if (ok) break;
                        if (++spins > 16u * a.spin_limit) {
                            atomicOr(a.flag, FLAG_COPY_TIMEOUT);
                            dead = true;
                            return;
                        }
                    }
                }
                mbar_expect_tx(&sm.full[stage], DG_STAGE * DG_BOX_BYTES);
                bulk_g2s(sm.ring[stage * DG_STAGE], src, DG_STAGE * DG_BOX_BYTES, &sm.full[stage]);
                ++i;
            };
            const int spl = strm.boxes_per_layer / DG_STAGE;   // stages per layer
            for (int pos = 0; pos < n_pos; ++pos) {
                for (int l = 0; l < a.n_layers; ++l) {
                    const unsigned char* src = strm.layers + (size_t)(l * DG_CL + c) * strm.boxes_per_layer * DG_BOX_BYTES;
                    for (int sg = 0; sg < spl; ++sg) issue_stage(src + (size_t)sg * DG_STAGE * DG_BOX_BYTES);
                }
                if (pos >= 1) {
                    const unsigned char* src = strm.head + (size_t)((pos - 1) * DG_CL + c) * 32 * DG_BOX_BYTES;
                    for (int sg = 0; sg < 32 / DG_STAGE; ++sg) issue_stage(src + (size_t)sg * DG_STAGE * DG_BOX_BYTES);
                }
            }
        }
        __syncwarp();
        cluster_wait();
        return;
    }

    // ------------------------------------------------------------------ consumers (256 threads)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
    pdl_wait();
    cluster_wait();
    const int set = warp >> 2, mt = warp & 3;   // warp set (even / odd boxes of a row group), 16-row tile of the box
    const int g = lane >> 2, t = lane & 3;
    DgState st{0, 0, false, -1, a.flag, a.spin_limit};
    unsigned ph_rs = 0, ph_ag = 0, ph_lg = 0, ph_x = 0;

    for (int pos = 0; pos < n_pos; ++pos) {
        // ---- the position's token rows
        if (pos >= 2) {
            dg_wait_or_die(st, &sm.bar_x, ph_x & 1);
            ++ph_x;
        }
        for (int e = tid; e < R * (DG_D / 8); e += DG_CONSUMERS) {
            const int n = e / (DG_D / 8), k = (e % (DG_D / 8)) * 8;
            const int b = b0 + (n < n_valid ? n : 0);
            const bf16* src = pos < 2 ? a.x2 + ((size_t)b * 2 + pos) * DG_D : a.x1 + (size_t)b * DG_D;
            *reinterpret_cast<uint4*>(&sm.x[n][k]) = __ldcg(reinterpret_cast<const uint4*>(src + k));
        }
        dg_bar();
        for (int l = 0; l < a.n_layers; ++l) {
            bf16* kcl = a.kc + (size_t)l * a.max_rows * a.Q * DG_D;
            bf16* vcl = a.vc + (size_t)l * a.max_rows * a.Q * DG_D;
            unsigned long long* dbg = (pos == 8 && l == 1) ? a.dbg : nullptr;
            fb_stamp(dbg, 0);
            dg_norm<R>(sm, a.attn_norm[l], a.eps);
            dg_bar();
            fb_stamp(dbg, 1);
            // ---- q, k, v rows of head c: q is the first warp set's, k the second's (both row groups fit the ring at
            // once), v is split over K between them; one hand-over instead of three
            for (int rg = 0; rg < 3; ++rg) {
                float acc[NT][4], oth[NT][4];
                bool mine;
                if (rg < 2) {
                    dg_rowgroup<R>(sm, st, 8, &sm.h[0][0], DG_XS, 0, 64, acc, rg);
                    mine = set == rg;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) oth[nt][0] = oth[nt][1] = oth[nt][2] = oth[nt][3] = 0.f;
                } else {
                    dg_rowgroup<R>(sm, st, 8, &sm.h[0][0], DG_XS, 0, 64, acc);
                    mine = dg_combine<R>(sm, st, acc, oth);
                }
                if (mine) {
                    float (*dst)[HD] = rg == 0 ? sm.q : (rg == 1 ? sm.kn : sm.vn);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int n = nt * 8 + 2 * t + (i & 1), dim = mt * 16 + g + (i >> 1) * 8;
                            const float v = rbf(acc[nt][i] + oth[nt][i]);
                            dst[n][dim] = v;
                            if (rg > 0 && n < n_valid) {
                                bf16* cache = rg == 1 ? kcl : vcl;
                                cache[((size_t)(b0 + n) * a.Q + pos) * DG_D + c * HD + dim] = f2bf(v);
                            }
                        }
                }
            }
            dg_bar();
            fb_stamp(dbg, 2);
            // ---- attention of head c: one warp per stream, keys [0, pos) from the scratch + the new key
            for (int n = warp; n < R; n += DG_CONSUMERS / 32) {
                const int s8 = lane & 7, g4 = lane >> 3;
                const int b = b0 + (n < n_valid ? n : 0);
                const bf16* kb = kcl + (size_t)b * a.Q * DG_D + c * HD + s8 * 8;
                const bf16* vb = vcl + (size_t)b * a.Q * DG_D + c * HD + s8 * 8;
                uint4 kr[4], vr[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int tk = u * 4 + g4;
                    const bool ok = tk < pos;
                    kr[u] = ok ? __ldcg(reinterpret_cast<const uint4*>(kb + (size_t)tk * DG_D)) : make_uint4(0, 0, 0, 0);
                    vr[u] = ok ? __ldcg(reinterpret_cast<const uint4*>(vb + (size_t)tk * DG_D)) : make_uint4(0, 0, 0, 0);
                }
                float qf[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) qf[j] = sm.q[n][s8 * 8 + j];
                float m = NEG_BIG, lsum = 0.f, acc8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc8[j] = 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (u * 4 < pos) {  // uniform over the warp
                        float kf[8], vf[8];
                        unpack8(kr[u], kf);
                        unpack8(vr[u], vf);
                        float d = 0.f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) d = fmaf(qf[j], kf[j], d);
                        d += __shfl_xor_sync(0xffffffffu, d, 1);
                        d += __shfl_xor_sync(0xffffffffu, d, 2);
                        d += __shfl_xor_sync(0xffffffffu, d, 4);
                        if (u * 4 + g4 < pos) {
                            const float sc = d * 0.125f;
                            const float mn = fmaxf(m, sc);
                            const float corr = __expf(m - mn), p = __expf(sc - mn);
                            lsum = lsum * corr + p;
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc8[j] = fmaf(p, vf[j], acc8[j] * corr);
                            m = mn;
                        }
                    }
                }
#pragma unroll
                for (int o = 8; o <= 16; o <<= 1) {
                    const float mo = __shfl_xor_sync(0xffffffffu, m, o);
                    const float lo = __shfl_xor_sync(0xffffffffu, lsum, o);
                    float ao[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) ao[j] = __shfl_xor_sync(0xffffffffu, acc8[j], o);
                    softmax_merge(m, lsum, acc8, mo, lo, ao);
                }
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) d = fmaf(qf[j], sm.kn[n][s8 * 8 + j], d);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                const float sc = d * 0.125f;
                const float mn = fmaxf(m, sc);
                const float corr = __expf(m - mn), p = __expf(sc - mn);
                lsum = lsum * corr + p;
                if (g4 == 0) {
                    const float inv = 1.f / lsum;
                    float o8[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o8[j] = fmaf(p, sm.vn[n][s8 * 8 + j], acc8[j] * corr) * inv;
                    *reinterpret_cast<uint4*>(&sm.attn[n][s8 * 8]) = pack8(o8);
                }
            }
            dg_bar();
            fb_stamp(dbg, 3);
            // ---- this head's K-slice of out_proj, all 512 output rows
            for (int rb = 0; rb < 8; ++rb) {   // row blocks alternate between the warp sets
                float acc[NT][4];
                dg_rowgroup<R>(sm, st, 1, &sm.attn[0][0], DG_AS, 0, 0, acc, rb & 1);
                if (set == (rb & 1)) dg_push_partial<R>(sm, c, rb, acc);
            }
            fb_stamp(dbg, 4);
            dg_residual_exchange<R>(sm, st, c, ph_rs, ph_ag);
            fb_stamp(dbg, 5);
            // ---- MLP: this CTA's hidden units
            dg_norm<R>(sm, a.mlp_norm[l], a.eps);
            dg_bar();
            fb_stamp(dbg, 6);
            for (int ub = 0; ub < n_ub; ++ub) {
                // w1's row group is the first warp set's, w3's the second's (both fit the ring at once, and a warp
                // waits for its own two stage fills only); the second set hands its sums over for the gate product
                float acc[NT][4], a3[NT][4], oth[NT][4];
                dg_rowgroup<R>(sm, st, 8, &sm.h[0][0], DG_XS, 0, 64, acc, 0);
                dg_rowgroup<R>(sm, st, 8, &sm.h[0][0], DG_XS, 0, 64, a3, 1);
                if (dg_combine<R>(sm, st, a3, oth)) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int n = nt * 8 + 2 * t + (i & 1), u = ub * 64 + mt * 16 + g + (i >> 1) * 8;
                            const float a1 = rbf(acc[nt][i]), a3 = rbf(oth[nt][i]);
                            const float sl = rbf(a1 / (1.0f + expf(-a1)));
                            sm.g[n][u] = u < a.upc ? f2bf(sl * a3) : f2bf(0.f);
                        }
                }
            }
            dg_bar();
            fb_stamp(dbg, 7);
            for (int rb = 0; rb < 8; ++rb) {   // a row block's boxes all go to one warp set: no combine, no barrier
                float acc[NT][4];
                dg_rowgroup<R>(sm, st, n_ub, &sm.g[0][0], DG_GS, 0, 64, acc, rb & 1);
                if (set == (rb & 1)) dg_push_partial<R>(sm, c, rb, acc);
            }
            fb_stamp(dbg, 8);
            dg_residual_exchange<R>(sm, st, c, ph_rs, ph_ag);
            fb_stamp(dbg, 9);
        }
        if (pos == 0) continue;
        unsigned long long* dbg = pos == 8 ? a.dbg : nullptr;
        fb_stamp(dbg, 10);
        // ---- head of codebook `pos`: this CTA's 256 rows, then sampling of stream c (c + 8, ...)
        dg_norm<R>(sm, a.final_norm, a.eps);
        dg_bar();
        for (int rb = 0; rb < 4; ++rb) {
            float acc[NT][4];
            dg_rowgroup<R>(sm, st, 8, &sm.h[0][0], DG_XS, 0, 64, acc, rb & 1);
            if (set == (rb & 1)) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int n = nt * 8 + 2 * t + (i & 1), row = c * 256 + rb * 64 + mt * 16 + g + (i >> 1) * 8;
                        if (n < n_valid) {
                            const bf16 o = f2bf(acc[nt][i]);
                            a.logits[(size_t)(b0 + n) * a.CS + row] = o;
                            if (a.tap) a.tap[(size_t)(b0 + n) * (a.Q - 1) * a.CS + (size_t)(pos - 1) * a.CS + row] = o;
                        }
                    }
            }
        }
        fb_stamp(dbg, 11);
        __threadfence();
        dg_bar();
        if (tid == 0)
            for (int p = 0; p < DG_CL; ++p) remote_arrive(&sm.bar_logits, p);
        dg_wait_or_die(st, &sm.bar_logits, ph_lg & 1);
        ++ph_lg;
        fb_stamp(dbg, 12);
        for (int n = c; n < n_valid; n += DG_CL) {
            SampleArgs sa = a.sa;
            sa.logits = a.logits;
            sa.stride = a.CS;
            sa.codebook = pos;
            sa.out_col = pos;
            sa.first_frame = 0;
            sa.bump_frame = pos == n_pos - 1;
            sa.zero_from = 0;
            sa.eos_logit = nullptr;
            sa.eos_prob = nullptr;
            sa.stats_out = nullptr;
            sa.emb_out = pos + 1 < n_pos ? a.x1 : nullptr;
            sa.emb_p = pos + 1;
            sa.emb_row_mul = 1;
            sa.emb_row_add = 0;
            sample_row(sa, b0 + n, tid, sm.samp, 1);
            dg_bar();
        }
        fb_stamp(dbg, 13);
        if (pos + 1 < n_pos) {  // the last position's peers may already have retired: nothing is sent to them
            __threadfence();
            dg_bar();
            if (tid == 0)
                for (int p = 0; p < DG_CL; ++p) remote_arrive(&sm.bar_x, p);
        }
    }
}

}  // namespace vuib
