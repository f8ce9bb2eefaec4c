// One whole decode frame as ONE persistent kernel (up to 8 streams): the embed
// gather-sum, 24 backbone blocks, final norm + heads, cb0 sampling, the depth
// transformer over the remaining codebooks and the token that feeds the next
// codebook, separated by grid-wide barriers instead of kernel launches.
//
// One CTA per SM, launched cooperatively so that all CTAs are resident.  A warp
// fetches the weight rows of its NEXT phase before it arrives at the barrier that
// ends the current one, so the HBM round trip of the weights overlaps the barrier
// and only the (L2-resident) activations are read after it.  The arithmetic is
// that of the per-phase kernels in decode_kernels.cuh, functor for functor, so
// both paths produce identical bits.
//
// Barrier: one 32-bit counter, zeroed by the host before the launch; arrival is a
// red.release, the wait an ld.acquire poll with an iteration limit.  On a timeout
// the CTA records FLAG_BARRIER_TIMEOUT, stops waiting for the rest of the launch
// and runs to the end, so a lost CTA can never hang the GPU.
#pragma once
#include "../../include/vuib200.h"
#include "decode_kernels.cuh"

namespace vuib {

constexpr int PF_THREADS = 256;
constexpr int PF_WARPS = PF_THREADS / 32;
constexpr int PF_ATT_GROUPS = PF_THREADS / ATT_THREADS;
constexpr unsigned BAR_SPIN_LIMIT = 1u << 21;  // ~1 s of polling at ~0.5 us per poll
constexpr int FLAG_BARRIER_TIMEOUT = 8;
constexpr int TRACE_MAX = 1024;  // barrier records kept per launch

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

struct DevModel {   // device-resident copy of the bound pointers
    VuibWeights w;
    void* k[VUIB_MAX_LAYERS];
    void* v[VUIB_MAX_LAYERS];
    const bf16* rope;
    int32_t* seq_lens;
};

struct FrameBufs {  // workspace regions
    int32_t *row_slot, *row_pos;
    bf16 *x, *q, *attn, *act;
    float* part;
    int32_t* counters;
    bf16 *rq_x2, *rq_x, *rq_q, *rq_act, *rq_k, *rq_v, *rq_logits;
    int32_t* code_cur;
    SamplingCtl* ctl;
    int32_t* frame_ctr;
    float* rep_counts;
    int32_t *rep_hist, *rep_head, *rep_filled;
    int32_t* flag;
    unsigned* bar;
    unsigned long long* trace;  // [0] = entries written; then (arrive, release) globaltimer pairs of CTA 0
};

struct FrameArgs {
    const DevModel* m;
    FrameBufs b;
    int B;
    const int32_t* slots;
    const int32_t* seq_inc;
    int64_t* codes_io;
    bf16 *hidden_out, *cb0_out, *eos_out;
    float* eos_prob;
    bf16 *tap_layers, *tap_rq;
    int n_layers, n_heads, n_kv_heads, max_seq, n_slots, S;
    int Q, CS, rq_n_layers, rq_n_heads, max_rows;
    float norm_eps, rq_norm_eps;
    int n_codebooks;   // codes to emit (Q' <= Q)
    int do_backbone;   // 0: depth step only (hidden_out / cb0_out / eos_out are inputs)
    int first_frame;
};

struct GridBarrier {
    unsigned* counter;
    unsigned target;
    unsigned n;
    int32_t* flag;
    bool dead;
    unsigned long long* trace;  // CTA 0 only, may be NULL
    unsigned n_sync;
    __device__ __forceinline__ void sync() {
        __syncthreads();
        if (threadIdx.x == 0) {
            target += n;
            const bool rec = trace && blockIdx.x == 0 && n_sync < TRACE_MAX;
            if (rec) trace[1 + 2 * n_sync] = globaltimer_ns();
            // release: the bar.sync above ordered the CTA's writes before this thread
            asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(counter), "r"(1u) : "memory");
            if (!dead) {
                unsigned v, spins = 0;
                for (;;) {
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
                    if ((int)(v - target) >= 0) break;
                    if (++spins > BAR_SPIN_LIMIT) {
                        atomicOr(flag, FLAG_BARRIER_TIMEOUT);
                        dead = true;
                        break;
                    }
                }
            }
            if (rec) {
                trace[2 + 2 * n_sync] = globaltimer_ns();
                trace[0] = n_sync + 1;
            }
            ++n_sync;
        }
        __syncthreads();
    }
};

template <int K, class Epi>
struct WPref {
    uint4 w[Epi::NC][(K + 255) / 256];
};

template <int K, class Epi>
__device__ __forceinline__ void wload(const Epi& ep, int item, WPref<K, Epi>& p) {
    constexpr int IT = (K + 255) / 256;
    const int lane = threadIdx.x & 31;
    const bf16* wr[Epi::NC];
    ep.rows(item, wr);
#pragma unroll
    for (int c = 0; c < Epi::NC; ++c)
#pragma unroll
        for (int it = 0; it < IT; ++it) {
            const int k = it * 256 + lane * 8;
            p.w[c][it] = (k < K) ? ldg_stream(wr[c] + k) : make_uint4(0, 0, 0, 0);
        }
}

// Fetch the weight rows of this warp's first item of a phase (before the barrier).
template <int K, class Epi>
__device__ __forceinline__ void wprefetch(const Epi& ep, int n_items, WPref<K, Epi>& p) {
    const int item = blockIdx.x * PF_WARPS + (threadIdx.x >> 5);
    if (item < n_items) wload<K, Epi>(ep, item, p);
}

template <int K, int RT, class Stage, class Epi>
__device__ __forceinline__ void gemv_phase(const Stage& st, const Epi& ep, int M, int n_items,
                                           bf16* Xs, WPref<K, Epi>& p) {
    constexpr int NC = Epi::NC;
    constexpr int IT = (K + 255) / 256;
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * PF_WARPS + (threadIdx.x >> 5), tw = gridDim.x * PF_WARPS;
    for (int r0 = 0; r0 < M; r0 += RT) {
        const int nr = min(RT, M - r0);
        if (r0) __syncthreads();
        st.template stage<K>(Xs, r0, nr);
        __syncthreads();
        int nth = 0;
        for (int item = gw; item < n_items; item += tw, ++nth) {
            if (nth > 0 || (r0 > 0 && n_items > tw)) wload<K, Epi>(ep, item, p);
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
                    for (int c = 0; c < NC; ++c) unpack8(p.w[c][it], wf[c]);
#pragma unroll
                    for (int r = 0; r < RT; ++r) {
                        if (r < nr) {
                            float xf[8];
                            unpack8(*reinterpret_cast<const uint4*>(Xs + r * K + k), xf);
#pragma unroll
                            for (int c = 0; c < NC; ++c)
#pragma unroll
                                for (int j = 0; j < 8; ++j) acc[c][r] = fmaf(wf[c][j], xf[j], acc[c][r]);
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int r = 0; r < RT; ++r) acc[c][r] = warp_sum(acc[c][r]);
            ep.template store<RT>(item, r0, nr, lane, acc);
        }
    }
}

// Depth token for position p: code_emb[(p-1)*CS + code] + pos_emb[p], by threads 0..63.
__device__ __forceinline__ void rq_embed_row(int code, const bf16* code_emb, const bf16* pos_emb,
                                             bf16* out_row, int rd, int CS, int p, int tid) {
    const bf16* e = code_emb + ((size_t)(p - 1) * CS + code) * rd;
    const bf16* pe = pos_emb + (size_t)p * rd;
    for (int k = tid * 8; k < rd; k += SAMPLE_THREADS * 8) {
        float a[8], c[8], s[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(e + k)), a);
        unpack8(__ldg(reinterpret_cast<const uint4*>(pe + k)), c);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] = a[j] + c[j];
        *reinterpret_cast<uint4*>(out_row + k) = pack8(s);
    }
}

template <int RT, int RQF>
__device__ __forceinline__ void rq_layers_phase(const FrameArgs& a, GridBarrier& bar, bf16* Xs, int M,
                                                bf16* x, int rows_per_b, int pos_base) {
    constexpr int RD = 512;
    const DevModel& m = *a.m;
    const FrameBufs& b = a.b;
    const size_t layer_kv = (size_t)a.max_rows * a.Q * RD;
    for (int li = 0; li < a.rq_n_layers; ++li) {
        bf16* kc = b.rq_k + li * layer_kv;
        bf16* vc = b.rq_v + li * layer_kv;
        EpiQkv eq{static_cast<const bf16*>(m.w.rq_wqkv[li]), RD, b.rq_q, RD, RD, kc, vc,
                  nullptr, nullptr, a.Q, nullptr, rows_per_b, pos_base, 0};
        WPref<RD, EpiQkv> wq;
        wprefetch<RD>(eq, 3 * RD / 2, wq);
        bar.sync();
        StageNorm sn{x, static_cast<const bf16*>(m.w.rq_attn_norm[li]), a.rq_norm_eps, 1, 0};
        gemv_phase<RD, RT>(sn, eq, M, 3 * RD / 2, Xs, wq);

        EpiResidual eo{static_cast<const bf16*>(m.w.rq_out_proj[li]), RD, x, RD, nullptr};
        WPref<RD, EpiResidual> wo;
        wprefetch<RD>(eo, RD, wo);
        bar.sync();
        StageRqAttn sa{b.rq_q, kc, vc, a.rq_n_heads, a.Q, rows_per_b, pos_base};
        gemv_phase<RD, RT>(sa, eo, M, RD, Xs, wo);

        EpiSwiGLU eg{static_cast<const bf16*>(m.w.rq_w1[li]), static_cast<const bf16*>(m.w.rq_w3[li]), RD,
                     b.rq_act, RQF};
        WPref<RD, EpiSwiGLU> wg;
        wprefetch<RD>(eg, RQF, wg);
        bar.sync();
        StageNorm sm{x, static_cast<const bf16*>(m.w.rq_mlp_norm[li]), a.rq_norm_eps, 1, 0};
        gemv_phase<RD, RT>(sm, eg, M, RQF, Xs, wg);

        EpiResidual ew{static_cast<const bf16*>(m.w.rq_w2[li]), RQF, x, RD, nullptr};
        WPref<RQF, EpiResidual> ww;
        wprefetch<RQF>(ew, RD, ww);
        bar.sync();
        StageCopy sc{b.rq_act};
        gemv_phase<RQF, RT>(sc, ew, M, RD, Xs, ww);
    }
}

template <int RT, int RQF>
__global__ void __launch_bounds__(PF_THREADS, 1) k_frame(FrameArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Xs = reinterpret_cast<bf16*>(smem_raw);
    __shared__ AttnSmem att_sm[PF_ATT_GROUPS];
    __shared__ SampleSmem samp_sm;
    constexpr int D = 1024, F = 3072, RD = 512;
    const DevModel& m = *a.m;
    const FrameBufs& b = a.b;
    GridBarrier bar{b.bar, 0u, gridDim.x, b.flag, false, b.trace, 0u};
    const int B = a.B, cta = blockIdx.x, tid = threadIdx.x;
    const int qc = a.n_heads * HD, kvc = a.n_kv_heads * HD;

    if (a.do_backbone) {
        // ---- embed: CTA r gathers and sums the 16 table rows of stream r --------------
        if (cta < B) {
            const int r = cta;
            int slot = a.slots[r];
            if (slot < 0 || slot >= a.n_slots) {
                if (tid == 0) atomicOr(b.flag, FLAG_BAD_SLOT);
                slot = a.n_slots - 1;
            }
            if (tid == 0) {
                int pos = m.seq_lens[slot];
                if (pos < 0 || pos >= a.max_seq) {
                    atomicOr(b.flag, FLAG_BAD_POS);
                    pos = pos < 0 ? 0 : a.max_seq - 1;
                }
                b.row_slot[r] = slot;
                b.row_pos[r] = pos;
            }
            const bf16* table = static_cast<const bf16*>(m.w.audio_emb);
            for (int k = tid * 8; k < D; k += PF_THREADS * 8) {
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                for (int q = 0; q < a.Q; ++q) {
                    long long c = a.codes_io[(size_t)r * a.Q + q];
                    if (c < 0 || c >= a.CS) {
                        atomicOr(b.flag, FLAG_BAD_CODE);
                        c = 0;
                    }
                    float f[8];
                    unpack8(__ldg(reinterpret_cast<const uint4*>(table + ((size_t)q * a.CS + c) * D + k)), f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += f[j];
                }
                *reinterpret_cast<uint4*>(b.x + (size_t)r * D + k) = pack8(acc);
            }
        }
        for (int li = 0; li < a.n_layers; ++li) {
            EpiQkv eq{static_cast<const bf16*>(m.w.wqkv[li]), D, b.q, qc, kvc,
                      static_cast<bf16*>(m.k[li]), static_cast<bf16*>(m.v[li]),
                      b.row_slot, b.row_pos, a.max_seq, m.rope, 1, 0, 0};
            WPref<D, EpiQkv> wq;
            wprefetch<D>(eq, (qc + 2 * kvc) / 2, wq);
            bar.sync();
            StageNorm sn{b.x, static_cast<const bf16*>(m.w.attn_norm[li]), a.norm_eps, 1, 0};
            gemv_phase<D, RT>(sn, eq, B, (qc + 2 * kvc) / 2, Xs, wq);

            EpiResidual eo{static_cast<const bf16*>(m.w.out_proj[li]), D, b.x, D, nullptr};
            WPref<D, EpiResidual> wo;
            wprefetch<D>(eo, D, wo);
            bar.sync();
            {   // attention: a group of 128 threads per (split, kv head, row) unit
                AttnArgs aa{b.q, static_cast<const bf16*>(m.k[li]), static_cast<const bf16*>(m.v[li]),
                            b.row_slot, b.row_pos, b.part, b.counters, b.attn,
                            a.n_heads, a.n_kv_heads, a.max_seq, a.S,
                            (b.trace && cta == 1 && li == 5 && tid < ATT_THREADS) ? b.trace + 1 + 2 * TRACE_MAX : nullptr};
                const int group = tid / ATT_THREADS, gt = tid % ATT_THREADS;
                const int units = a.S * a.n_kv_heads * B;
                for (int u = cta * PF_ATT_GROUPS + group; u < units; u += gridDim.x * PF_ATT_GROUPS) {
                    bar_named(1 + group, ATT_THREADS);
                    attn_unit(aa, u % a.S, (u / a.S) % a.n_kv_heads, u / (a.S * a.n_kv_heads), gt,
                              att_sm[group], 1 + group);
                }
            }
            bar.sync();
            StageCopy sc{b.attn};
            gemv_phase<D, RT>(sc, eo, B, D, Xs, wo);

            EpiSwiGLU eg{static_cast<const bf16*>(m.w.w1[li]), static_cast<const bf16*>(m.w.w3[li]), D,
                         b.act, F};
            WPref<D, EpiSwiGLU> wg;
            wprefetch<D>(eg, F, wg);
            bar.sync();
            StageNorm sm{b.x, static_cast<const bf16*>(m.w.mlp_norm[li]), a.norm_eps, 1, 0};
            gemv_phase<D, RT>(sm, eg, B, F, Xs, wg);

            bf16* tap = a.tap_layers ? a.tap_layers + (size_t)li * a.max_rows * D : nullptr;
            EpiResidual ew{static_cast<const bf16*>(m.w.w2[li]), F, b.x, D, tap};
            WPref<F, EpiResidual> ww;
            wprefetch<F>(ew, D, ww);
            bar.sync();
            StageCopy sa{b.act};
            gemv_phase<F, RT>(sa, ew, B, D, Xs, ww);
        }
        // ---- final norm + codec_head + eos_head ----------------------------------------
        {
            EpiLogits el{static_cast<const bf16*>(m.w.codec_head), D, a.CS, a.cb0_out,
                         static_cast<const bf16*>(m.w.eos_w), static_cast<const bf16*>(m.w.eos_b), a.eos_out,
                         nullptr, 0};
            WPref<D, EpiLogits> wh;
            wprefetch<D>(el, a.CS + 1, wh);
            bar.sync();
            StageNorm sf{b.x, static_cast<const bf16*>(m.w.final_norm), a.norm_eps, 1, 0};
            gemv_phase<D, RT>(sf, el, B, a.CS + 1, Xs, wh);
            if (cta == 0) {  // B <= RT: the staged tile is the final-norm output of every row
                for (int i = tid; i < B * (D / 8); i += PF_THREADS)
                    reinterpret_cast<uint4*>(a.hidden_out)[i] = reinterpret_cast<const uint4*>(Xs)[i];
                if (tid < B) {
                    const int inc = a.seq_inc ? a.seq_inc[tid] : 1;
                    if (inc) m.seq_lens[__ldcg(b.row_slot + tid)] += inc;
                }
            }
        }
    }

    // ---- depth step ------------------------------------------------------------------
    const int Qn = a.n_codebooks;
    const bf16* pos_emb = static_cast<const bf16*>(m.w.rq_pos_emb);
    const bf16* code_emb = static_cast<const bf16*>(m.w.rq_code_emb);
    SampleArgs sa;
    sa.ctl = b.ctl;
    sa.slots = a.slots;
    sa.frame_ctr = b.frame_ctr;
    sa.rep_counts = b.rep_counts;
    sa.rep_hist = b.rep_hist;
    sa.rep_head = b.rep_head;
    sa.rep_filled = b.rep_filled;
    sa.code_cur = b.code_cur;
    sa.codes_out = a.codes_io;
    sa.Q = a.Q;
    sa.emb_out = nullptr;
    sa.stats_out = nullptr;
    {
        EpiProjPos ep{static_cast<const bf16*>(m.w.rq_backbone_proj), D, pos_emb, b.rq_x2, RD, 2};
        WPref<D, EpiProjPos> wp;
        wprefetch<D>(ep, RD, wp);
        bar.sync();
        if (cta < B && tid < SAMPLE_THREADS) {  // cb0, then depth position 1 from it
            sa.logits = a.cb0_out;
            sa.stride = a.CS;
            sa.codebook = 0;
            sa.out_col = 0;
            sa.first_frame = a.first_frame;
            sa.eos_logit = a.eos_out;
            sa.eos_prob = a.eos_prob;
            sa.bump_frame = 0;
            sa.zero_from = Qn < a.Q ? Qn : 0;
            const int code = sample_row(sa, cta, tid, samp_sm, 5);
            rq_embed_row(code, code_emb, pos_emb, b.rq_x2 + ((size_t)2 * cta + 1) * RD, RD, a.CS, 1, tid);
        }
        StageCopy sh{a.hidden_out};
        gemv_phase<D, RT>(sh, ep, B, RD, Xs, wp);
    }
    sa.eos_logit = nullptr;
    sa.eos_prob = nullptr;
    sa.first_frame = 0;
    sa.zero_from = 0;
    rq_layers_phase<RT, RQF>(a, bar, Xs, 2 * B, b.rq_x2, 2, 0);
    const bf16* head = static_cast<const bf16*>(m.w.rq_head);
    for (int i = 0; i < Qn - 1; ++i) {
        if (i > 0) rq_layers_phase<RT, RQF>(a, bar, Xs, B, b.rq_x, 1, i + 1);
        EpiLogits el{head + (size_t)i * a.CS * RD, RD, a.CS, b.rq_logits, nullptr, nullptr, nullptr,
                     a.tap_rq ? a.tap_rq + (size_t)i * a.CS : nullptr, (a.Q - 1) * a.CS};
        WPref<RD, EpiLogits> wh;
        wprefetch<RD>(el, a.CS, wh);
        bar.sync();
        StageNorm sn{i == 0 ? b.rq_x2 : b.rq_x, static_cast<const bf16*>(m.w.rq_norm), a.rq_norm_eps,
                     i == 0 ? 2 : 1, i == 0 ? 1 : 0};
        gemv_phase<RD, RT>(sn, el, B, a.CS, Xs, wh);
        bar.sync();
        if (cta < B && tid < SAMPLE_THREADS) {
            sa.logits = b.rq_logits;
            sa.stride = a.CS;
            sa.codebook = i + 1;
            sa.out_col = i + 1;
            sa.bump_frame = (i == Qn - 2);
            const int code = sample_row(sa, cta, tid, samp_sm, 5);
            if (i + 1 < Qn - 1)
                rq_embed_row(code, code_emb, pos_emb, b.rq_x + (size_t)cta * RD, RD, a.CS, i + 2, tid);
        }
    }
}

}  // namespace vuib
