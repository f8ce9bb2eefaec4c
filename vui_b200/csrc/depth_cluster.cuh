// The whole depth step (cb0 sampling + the RQ depth transformer over the remaining
// codebooks) for up to 4 streams as ONE kernel on ONE thread-block cluster of 16 CTAs.
//
// Why a cluster: at this size every matrix-vector product is a few hundred KB that depends on
// the previous one, so the step is a chain of ~300 dependent stages.  As separate launches each
// stage costs ~3 us; here the 16 CTAs exchange activations through distributed shared memory
// (st.shared::cluster into every peer's copy) and meet on the hardware cluster barrier (~0.2 us),
// while the 25.7 MB of depth-transformer weights stay L2-resident and are streamed by 16 SMs.
//
// Work split per layer (d = 512, 8 heads, ffn RQF):
//   qkv   : head h is owned by the CTA pair (2h, 2h+1): CTA 2h computes q_h and the first half of
//           k_h, CTA 2h+1 the rest of k_h and v_h; K/V go to the depth KV cache in global memory.
//   attn  : CTA 2h runs head h (<= 16 keys) and broadcasts its 64 outputs to all 16 CTAs.
//   out   : CTA c owns rows [32c, 32c+32): x += bf16(W attn), broadcast.
//   w1/w3 : CTA c owns hidden units [RQF/16 * c, ...): SiLU(w1 h) * (w3 h), broadcast.
//   w2    : CTA c owns rows [32c, 32c+32): x += bf16(W act), broadcast.
//   head  : CTA c owns 128 of the 2048 logits; greedy = per-CTA argmax + 16-candidate merge
//           (first index on ties), sampling = logits to global, CTA r draws for stream r.
// Every dot product uses the lane/k order and the butterfly reduction of the GEMV kernels, every
// rounding point is the same, so the codes, logits and KV written are bit-identical to the graph
// of per-phase kernels.
#pragma once
#include "frame_kernel.cuh"
#include "tc_gemm.cuh"

namespace vuib {

constexpr int DC_CTAS = 16;
constexpr int DC_THREADS = 1024;  // 32 warps: the step is bound by dependent dot-product latency, not bytes
constexpr int DC_WARPS = DC_THREADS / 32;
constexpr int DC_RD = 512;

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Store a 16-bit value at the same shared-memory offset in CTA `peer` of the cluster.
__device__ __forceinline__ void dsmem_st16(const void* local_smem, unsigned peer, unsigned short v) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_smem)), "r"(peer));
    asm volatile("st.shared::cluster.u16 [%0], %1;" ::"r"(ra), "h"(v) : "memory");
}

__device__ __forceinline__ void dsmem_st32(const void* local_smem, unsigned peer, uint32_t v) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_smem)), "r"(peer));
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(ra), "r"(v) : "memory");
}

struct DepthArgs {
    const DevModel* m;
    FrameBufs b;
    int B;
    const int32_t* slots;
    const bf16* hidden;      // (B, 1024) final-norm backbone output
    const bf16* cb0_logits;  // (B, CS)
    const bf16* eos_logit;   // (B) or NULL
    float* eos_prob;         // (B) or NULL
    int64_t* codes_out;      // (B, Q)
    bf16* tap_rq;
    int Q, CS, rq_n_layers, rq_n_heads, max_rows;
    float rq_norm_eps;
    int n_codebooks, first_frame;
    unsigned long long* dbg;  // optional device-clock stamps (profiling aid): pass 2, layer 0
};

__device__ __forceinline__ void dc_stamp(const DepthArgs& a, int p, int li, int i) {
    if (a.dbg && p == 2 && li == 0 && threadIdx.x == 0 && cluster_rank() == 0) a.dbg[i] = globaltimer_ns();
}

// RMSNorm of the RT rows in shared memory (same arithmetic as StageNorm): warp r -> row r.
template <int RT>
__device__ __forceinline__ void dc_norm(const bf16* xs, const bf16* w, float eps, bf16* out, int B) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < B; r += DC_WARPS) {
        float v[2][8];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            unpack8(*reinterpret_cast<const uint4*>(xs + r * DC_RD + it * 256 + lane * 8), v[it]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[it][j], v[it][j], ss);
        }
        ss = warp_sum(ss);
        const float rinv = rsqrtf(ss / (float)DC_RD + eps);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            float wf[8], o[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(w + it * 256 + lane * 8)), wf);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rbf(v[it][j] * rinv) * wf[j];
            *reinterpret_cast<uint4*>(out + r * DC_RD + it * 256 + lane * 8) = pack8(o);
        }
    }
}

// One weight row (K bf16, row-major) against the RT activation rows in shared memory, with
// the row's 16-byte pieces already in registers.  Lane/k order and reduction as in k_gemv.
template <int K, int RT>
__device__ __forceinline__ void dc_dot(const uint4 (&w)[(K + 255) / 256], const bf16* Xs, int B, float (&acc)[RT]) {
    constexpr int IT = (K + 255) / 256;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.f;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        const int k = it * 256 + lane * 8;
        if (k < K) {
            float wf[8];
            unpack8(w[it], wf);
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                if (r < B) {
                    float xf[8];
                    unpack8(*reinterpret_cast<const uint4*>(Xs + r * K + k), xf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[r] = fmaf(wf[j], xf[j], acc[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = warp_sum(acc[r]);
}

template <int K>
__device__ __forceinline__ void dc_load_row(const bf16* row, uint4 (&w)[(K + 255) / 256]) {
    constexpr int IT = (K + 255) / 256;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        const int k = it * 256 + lane * 8;
        w[it] = (k < K) ? ldg_stream(row + k) : make_uint4(0, 0, 0, 0);
    }
}

template <int RT, int RQF>
__global__ void __launch_bounds__(DC_THREADS, 1) k_depth_cluster(DepthArgs a) {
    constexpr int RD = DC_RD, D = 1024;
    constexpr int UPC = RQF / DC_CTAS;  // hidden units per CTA (88 or 96)
    __shared__ __align__(16) bf16 xs[RT * RD];      // residual stream (replicated in every CTA)
    __shared__ __align__(16) bf16 hs[RT * RD];      // normalised rows (local)
    __shared__ __align__(16) bf16 att[RT * RD];     // attention output (replicated)
    __shared__ __align__(16) bf16 big[RT * (RQF > D ? RQF : D)];  // SwiGLU activations (replicated) / hidden at p = 0
    __shared__ __align__(16) bf16 qs[RT * 64];      // q of this CTA's head (even CTAs)
    __shared__ float cand_v[DC_CTAS * RT];
    __shared__ int cand_i[DC_CTAS * RT];
    __shared__ int code_s[RT];
    __shared__ float wbest_v[DC_WARPS * RT];
    __shared__ int wbest_i[DC_WARPS * RT];
    __shared__ SampleSmem samp_sm;

    const DevModel& m = *a.m;
    const FrameBufs& b = a.b;
    const int B = a.B, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned c = cluster_rank();
    const int Qn = a.n_codebooks;
    const bf16* pos_emb = static_cast<const bf16*>(m.w.rq_pos_emb);
    const bf16* code_emb = static_cast<const bf16*>(m.w.rq_code_emb);
    const size_t layer_kv = (size_t)a.max_rows * a.Q * RD;
    pdl_trigger();
    pdl_wait();
    const SamplingCtl ctl = *b.ctl;

    SampleArgs sa;
    sa.ctl = b.ctl;
    sa.slots = a.slots;
    sa.frame_ctr = b.frame_ctr;
    sa.rep_counts = b.rep_counts;
    sa.rep_hist = b.rep_hist;
    sa.rep_head = b.rep_head;
    sa.rep_filled = b.rep_filled;
    sa.code_cur = b.code_cur;
    sa.codes_out = a.codes_out;
    sa.Q = a.Q;
    sa.emb_out = nullptr;
    sa.stats_out = nullptr;

    // ---- cb0: CTA r draws for stream r and tells everyone ---------------------------------
    if ((int)c < B && tid < SAMPLE_THREADS) {
        sa.logits = a.cb0_logits;
        sa.stride = a.CS;
        sa.codebook = 0;
        sa.out_col = 0;
        sa.first_frame = a.first_frame;
        sa.eos_logit = a.eos_logit;
        sa.eos_prob = a.eos_prob;
        sa.bump_frame = 0;
        sa.zero_from = Qn < a.Q ? Qn : 0;
        const int code = sample_row(sa, (int)c, tid, samp_sm, 1);
        if (tid < DC_CTAS) dsmem_st32(&code_s[c], tid, (uint32_t)code);
    }
    sa.eos_logit = nullptr;
    sa.eos_prob = nullptr;
    sa.first_frame = 0;
    sa.zero_from = 0;
    // hidden rows -> big (for the projection of position 0)
    for (int i = tid; i < B * (D / 8); i += DC_THREADS)
        reinterpret_cast<uint4*>(big)[i] = __ldcg(reinterpret_cast<const uint4*>(a.hidden) + i);
    cluster_sync_all();

    for (int p = 0; p < Qn; ++p) {
        // ---- token of depth position p -> xs (replicated) ---------------------------------
        if (p == 0) {
            // backbone_proj(hidden) + pos_emb[0]: CTA c owns rows [32c, 32c+32), 4 per warp
            const bf16* W = static_cast<const bf16*>(m.w.rq_backbone_proj);
            constexpr int RPW = 32 / DC_WARPS > 0 ? 32 / DC_WARPS : 1;
            uint4 w[RPW][4];
#pragma unroll
            for (int i = 0; i < RPW; ++i) dc_load_row<D>(W + (size_t)(c * 32 + warp * RPW + i) * D, w[i]);
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const int n = c * 32 + warp * RPW + i;
                float acc[RT];
                dc_dot<D, RT>(w[i], big, B, acc);
                const float pe = bf2f(pos_emb[n]);
                if (lane < DC_CTAS) {
#pragma unroll
                    for (int r = 0; r < RT; ++r)
                        if (r < B) dsmem_st16(&xs[r * RD + n], lane, __bfloat16_as_ushort(f2bf(rbf(acc[r]) + pe)));
                }
            }
            cluster_sync_all();
        } else {
            // code_emb[(p-1)*CS + code] + pos_emb[p]: every CTA builds its own copy
            for (int i = tid; i < B * (RD / 8); i += DC_THREADS) {
                const int r = i / (RD / 8), k = (i % (RD / 8)) * 8;
                float e[8], pe[8], s[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(code_emb + ((size_t)(p - 1) * a.CS + code_s[r]) * RD + k)), e);
                unpack8(__ldg(reinterpret_cast<const uint4*>(pos_emb + (size_t)p * RD + k)), pe);
#pragma unroll
                for (int j = 0; j < 8; ++j) s[j] = e[j] + pe[j];
                *reinterpret_cast<uint4*>(xs + r * RD + k) = pack8(s);
            }
            __syncthreads();
        }

        for (int li = 0; li < a.rq_n_layers; ++li) {
            bf16* kc = b.rq_k + li * layer_kv;
            bf16* vc = b.rq_v + li * layer_kv;
            dc_stamp(a, p, li, 0);
            // ---- qkv of head h by the CTA pair (2h, 2h+1): 96 rows each, 12 per warp ---------
            dc_norm<RT>(xs, static_cast<const bf16*>(m.w.rq_attn_norm[li]), a.rq_norm_eps, hs, B);
            __syncthreads();
            {
                const int h = c >> 1, odd = c & 1;
                const bf16* W = static_cast<const bf16*>(m.w.rq_wqkv[li]);
                constexpr int QPW = 96 / DC_WARPS;  // rows per warp
                uint4 w[QPW][2];
                int nrow[QPW];
#pragma unroll
                for (int i = 0; i < QPW; ++i) {
                    const int j = warp * QPW + i;  // 0..95 inside this CTA's share
                    // even: q_h[0..63], k_h[0..31]; odd: k_h[32..63], v_h[0..63]
                    nrow[i] = odd ? (j < 32 ? RD + h * 64 + 32 + j : 2 * RD + h * 64 + (j - 32))
                                  : (j < 64 ? h * 64 + j : RD + h * 64 + (j - 64));
                    dc_load_row<RD>(W + (size_t)nrow[i] * RD, w[i]);
                }
#pragma unroll
                for (int i = 0; i < QPW; ++i) {
                    float acc[RT];
                    dc_dot<RD, RT>(w[i], hs, B, acc);
                    if (lane == 0) {
                        const int n = nrow[i];
#pragma unroll
                        for (int r = 0; r < RT; ++r) {
                            if (r >= B) continue;
                            const bf16 o = f2bf(acc[r]);
                            if (n < RD) qs[r * 64 + (n - h * 64)] = o;
                            else if (n < 2 * RD) kc[((size_t)r * a.Q + p) * RD + (n - RD)] = o;
                            else vc[((size_t)r * a.Q + p) * RD + (n - 2 * RD)] = o;
                        }
                    }
                }
            }
            dc_stamp(a, p, li, 1);
            cluster_sync_all();  // K/V of position p from both CTAs of the pair are visible
            dc_stamp(a, p, li, 2);
            // ---- attention of head h on CTA 2h: warp r -> row r; lane = (key group g, chunk s) --
            if ((c & 1) == 0) {
                const int h = c >> 1, s = lane & 7, g = lane >> 3;
                for (int r = warp; r < B; r += DC_WARPS) {
                    float qf[8];
                    unpack8(*reinterpret_cast<const uint4*>(qs + r * 64 + s * 8), qf);
                    float mx = NEG_BIG, l = 0.f, acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                    for (int t0 = 0; t0 <= p; t0 += 4) {
                        const int t = t0 + g;
                        const bool ok = t <= p;
                        const size_t off = ((size_t)r * a.Q + (ok ? t : 0)) * RD + h * HD + s * 8;
                        float kf[8], vf[8];
                        unpack8(__ldcg(reinterpret_cast<const uint4*>(kc + off)), kf);
                        unpack8(__ldcg(reinterpret_cast<const uint4*>(vc + off)), vf);
                        float d = 0.f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) d = fmaf(qf[j], kf[j], d);
                        d += __shfl_xor_sync(0xffffffffu, d, 1);
                        d += __shfl_xor_sync(0xffffffffu, d, 2);
                        d += __shfl_xor_sync(0xffffffffu, d, 4);
                        if (ok) {
                            const float sc = d * 0.125f;
                            const float mn = fmaxf(mx, sc);
                            const float corr = __expf(mx - mn), pr = __expf(sc - mn);
                            l = l * corr + pr;
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc[j] = fmaf(pr, vf[j], acc[j] * corr);
                            mx = mn;
                        }
                    }
#pragma unroll
                    for (int o = 8; o <= 16; o <<= 1) {
                        const float mo = __shfl_xor_sync(0xffffffffu, mx, o);
                        const float lo = __shfl_xor_sync(0xffffffffu, l, o);
                        const float mn = fmaxf(mx, mo);
                        const float ca = __expf(mx - mn), cb = __expf(mo - mn);
                        l = l * ca + lo * cb;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float ao = __shfl_xor_sync(0xffffffffu, acc[j], o);
                            acc[j] = acc[j] * ca + ao * cb;
                        }
                        mx = mn;
                    }
                    // lanes with g == 0 hold dims s*8..s*8+7; pairs of bf16 go to the 16 CTAs:
                    // lane (g, s) serves peers 4g..4g+3 with the values it fetches from lane s
                    const float inv = 1.f / l;
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[2 * j] * inv, acc[2 * j + 1] * inv);
                        packed[j] = *reinterpret_cast<uint32_t*>(&t2);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) packed[j] = __shfl_sync(0xffffffffu, packed[j], s);  // from g == 0
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const unsigned peer = g * 4 + q4;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            dsmem_st32(&att[r * RD + h * HD + s * 8 + 2 * j], peer, packed[j]);
                    }
                }
            }
            dc_stamp(a, p, li, 3);
            cluster_sync_all();
            dc_stamp(a, p, li, 4);
            // ---- out_proj rows [32c, 32c+32): x += bf16(W att), 4 rows per warp ----------------
            {
                const bf16* W = static_cast<const bf16*>(m.w.rq_out_proj[li]);
                constexpr int RPW = 32 / DC_WARPS > 0 ? 32 / DC_WARPS : 1;
                uint4 w[RPW][2];
#pragma unroll
                for (int i = 0; i < RPW; ++i) dc_load_row<RD>(W + (size_t)(c * 32 + warp * RPW + i) * RD, w[i]);
#pragma unroll
                for (int i = 0; i < RPW; ++i) {
                    const int n = c * 32 + warp * RPW + i;
                    float acc[RT];
                    dc_dot<RD, RT>(w[i], att, B, acc);
                    if (lane < DC_CTAS) {
#pragma unroll
                        for (int r = 0; r < RT; ++r)
                            if (r < B) {
                                const bf16 o = f2bf(bf2f(xs[r * RD + n]) + rbf(acc[r]));
                                dsmem_st16(&xs[r * RD + n], lane, __bfloat16_as_ushort(o));
                            }
                    }
                }
            }
            dc_stamp(a, p, li, 5);
            cluster_sync_all();
            dc_stamp(a, p, li, 6);
            // ---- w1/w3 of hidden units [UPC*c, UPC*(c+1)): SiLU(w1 h) * (w3 h), broadcast ----------
            dc_norm<RT>(xs, static_cast<const bf16*>(m.w.rq_mlp_norm[li]), a.rq_norm_eps, hs, B);
            __syncthreads();
            {
                const bf16* W1 = static_cast<const bf16*>(m.w.rq_w1[li]);
                const bf16* W3 = static_cast<const bf16*>(m.w.rq_w3[li]);
                constexpr int UPW = (UPC + DC_WARPS - 1) / DC_WARPS;  // units per warp (11 or 12)
                constexpr int HALF = (UPW + 1) / 2;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint4 w1[HALF][2], w3[HALF][2];
#pragma unroll
                    for (int i = 0; i < HALF; ++i) {
                        const int u = warp + DC_WARPS * (half * HALF + i);
                        if (half * HALF + i < UPW && u < UPC) {
                            dc_load_row<RD>(W1 + (size_t)(c * UPC + u) * RD, w1[i]);
                            dc_load_row<RD>(W3 + (size_t)(c * UPC + u) * RD, w3[i]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < HALF; ++i) {
                        const int u = warp + DC_WARPS * (half * HALF + i);
                        if (half * HALF + i < UPW && u < UPC) {
                            float a1[RT], a3[RT];
                            dc_dot<RD, RT>(w1[i], hs, B, a1);
                            dc_dot<RD, RT>(w3[i], hs, B, a3);
                            if (lane < DC_CTAS) {
#pragma unroll
                                for (int r = 0; r < RT; ++r)
                                    if (r < B) {
                                        const float x1 = rbf(a1[r]), g = rbf(a3[r]);
                                        const float sl = rbf(x1 / (1.0f + expf(-x1)));
                                        dsmem_st16(&big[r * RQF + c * UPC + u], lane, __bfloat16_as_ushort(f2bf(sl * g)));
                                    }
                            }
                        }
                    }
                }
            }
            dc_stamp(a, p, li, 7);
            cluster_sync_all();
            dc_stamp(a, p, li, 8);
            // ---- w2 rows [32c, 32c+32): x += bf16(W act), 4 rows per warp ---------------------------
            {
                const bf16* W = static_cast<const bf16*>(m.w.rq_w2[li]);
                constexpr int RPW = 32 / DC_WARPS > 0 ? 32 / DC_WARPS : 1;
                uint4 w[RPW][(RQF + 255) / 256];
#pragma unroll
                for (int i = 0; i < RPW; ++i) dc_load_row<RQF>(W + (size_t)(c * 32 + warp * RPW + i) * RQF, w[i]);
#pragma unroll
                for (int i = 0; i < RPW; ++i) {
                    const int n = c * 32 + warp * RPW + i;
                    float acc[RT];
                    dc_dot<RQF, RT>(w[i], big, B, acc);
                    if (lane < DC_CTAS) {
#pragma unroll
                        for (int r = 0; r < RT; ++r)
                            if (r < B) {
                                const bf16 o = f2bf(bf2f(xs[r * RD + n]) + rbf(acc[r]));
                                dsmem_st16(&xs[r * RD + n], lane, __bfloat16_as_ushort(o));
                            }
                    }
                }
            }
            dc_stamp(a, p, li, 9);
            cluster_sync_all();
            dc_stamp(a, p, li, 10);
        }
        if (p == 0) continue;  // position 0 only feeds the caches

        // ---- head p-1 -> code p: CTA c owns logits [128c, 128c+128), 16 per warp ------------------
        dc_norm<RT>(xs, static_cast<const bf16*>(m.w.rq_norm), a.rq_norm_eps, hs, B);
        __syncthreads();
        {
            const int i_head = p - 1;
            const bf16* W = static_cast<const bf16*>(m.w.rq_head) + (size_t)i_head * a.CS * RD;
            float best_v[RT];
            int best_i[RT];
#pragma unroll
            for (int r = 0; r < RT; ++r) { best_v[r] = -3.0e38f; best_i[r] = 0x7fffffff; }
            constexpr int HPW = 128 / DC_WARPS;                 // logits per warp
            constexpr int HB = HPW > 8 ? 8 : HPW;               // rows fetched per batch
#pragma unroll
            for (int half = 0; half < HPW / HB; ++half) {
                uint4 w[HB][2];
#pragma unroll
                for (int i = 0; i < HB; ++i) dc_load_row<RD>(W + (size_t)(c * 128 + warp * HPW + half * HB + i) * RD, w[i]);
#pragma unroll
                for (int i = 0; i < HB; ++i) {
                    const int n = c * 128 + warp * HPW + half * HB + i;
                    float acc[RT];
                    dc_dot<RD, RT>(w[i], hs, B, acc);
#pragma unroll
                    for (int r = 0; r < RT; ++r) {
                        const bf16 o = f2bf(acc[r]);
                        const float v = bf2f(o);
                        if (v > best_v[r]) { best_v[r] = v; best_i[r] = n; }  // ascending n: first index wins ties
                        if (lane == 0 && r < B) {
                            b.rq_logits[(size_t)r * a.CS + n] = o;
                            if (a.tap_rq) a.tap_rq[(size_t)r * (a.Q - 1) * a.CS + (size_t)i_head * a.CS + n] = o;
                        }
                    }
                }
            }
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < RT; ++r) { wbest_v[warp * RT + r] = best_v[r]; wbest_i[warp * RT + r] = best_i[r]; }
            }
        }
        __syncthreads();
        const bool last = (p == Qn - 1);
        if (ctl.top_k_rq == 1) {
            // greedy: CTA-local best (warps hold ascending index ranges), then 16 candidates per row
            if (tid < B) {
                float bv = wbest_v[tid];
                int bi = wbest_i[tid];
                for (int w = 1; w < DC_WARPS; ++w)
                    if (wbest_v[w * RT + tid] > bv) { bv = wbest_v[w * RT + tid]; bi = wbest_i[w * RT + tid]; }
                for (unsigned peer = 0; peer < DC_CTAS; ++peer) {
                    dsmem_st32(&cand_v[c * RT + tid], peer, __float_as_uint(bv));
                    dsmem_st32(&cand_i[c * RT + tid], peer, (uint32_t)bi);
                }
            }
            cluster_sync_all();
            if (tid < B) {
                float bv = cand_v[tid];
                int bi = cand_i[tid];
                for (int q = 1; q < DC_CTAS; ++q)
                    if (cand_v[q * RT + tid] > bv) { bv = cand_v[q * RT + tid]; bi = cand_i[q * RT + tid]; }
                code_s[tid] = bi;
                if (c == 0) {
                    b.code_cur[tid] = bi;
                    a.codes_out[(size_t)tid * a.Q + p] = (int64_t)bi;
                    if (last) b.frame_ctr[a.slots[tid]] += 1;
                }
            }
            __syncthreads();
        } else {
            // sampling: all 2048 logits of a row are in global memory; CTA r draws for stream r
            cluster_sync_all();
            if ((int)c < B && tid < SAMPLE_THREADS) {
                sa.logits = b.rq_logits;
                sa.stride = a.CS;
                sa.codebook = p;
                sa.out_col = p;
                sa.bump_frame = last ? 1 : 0;
                const int code = sample_row(sa, (int)c, tid, samp_sm, 1);
                if (tid < DC_CTAS) dsmem_st32(&code_s[c], tid, (uint32_t)code);
            }
            cluster_sync_all();
        }
    }
}

}  // namespace vuib
