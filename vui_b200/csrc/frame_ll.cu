// One whole frame (backbone, heads, depth step) for up to 4 streams as ONE persistent kernel
// WITHOUT grid barriers: activations travel between the phases as self-validating words.
//
// Every activation element that crosses CTAs is a 32-bit word { bf16 value | 16-bit tag << 16 } in a
// global (L2-resident) buffer.  The tag names the phase that produced the word; a consumer loads the
// words it needs with ld.relaxed.gpu and simply retries until all of them carry the tag it expects.
// A 4-byte store is indivisible, so a word is either the old one or the new one: the data is its own
// flag, there is no fence, no atomic and no barrier on the path, and the hand-over from one phase to
// the next costs one L2 round trip (measured: 1.1 us per phase for a 1024-element all-gather among
// 148 CTAs, against 1.9 us for an atomic-counter barrier followed by plain loads).
//
// Why overwriting a buffer a few phases later is safe: a CTA can only run phase n once every word of
// phase n-1 exists, i.e. once every CTA has finished computing phase n-1, which it does after it
// has staged that phase's inputs in shared memory.  So while anybody writes in phase n, nobody
// still reads what phase n-1 read.  Every buffer here is rewritten two or more phases after its
// last reader.
//
// Tags: tag(g) = g mod 65535 + 1 for a phase counter g that runs on from launch to launch (kept in
// the workspace); 0 never occurs, so zeroed memory is "not yet".  Within a run of launches of the
// same shape (streams, codebooks) every word that is read was written in the same launch and the
// previous version is one launch (a few hundred phases) old, so a stale word never carries the
// expected tag.  When the shape changes, words may be older; the launch then clears the buffers and
// passes one ordinary grid barrier before it starts.
//
// Arithmetic, work split and rounding points are those of the per-phase kernels (same functors for
// the matrix-vector products, same sampler), so codes, logits and KV are bit-identical to them.
// Every wait is bounded: on expiry the kernel raises a flag word, stops waiting anywhere, and ends.
#include "frame_ll.h"

namespace vuib {

constexpr int FLAG_LL_TIMEOUT = 32;
constexpr unsigned LL_SPIN_LIMIT = 1u << 20;  // ~1 s at ~1 us per poll

struct LLWait {
    int32_t* flag;
    bool dead;
};

__device__ __forceinline__ uint32_t ll_tag(uint32_t g) { return g % 65535u + 1u; }

__device__ __forceinline__ uint32_t ll_word(bf16 v, uint32_t tag) {
    return (uint32_t)__bfloat16_as_ushort(v) | (tag << 16);
}

__device__ __forceinline__ bf16 ll_val(uint32_t w) { return __ushort_as_bfloat16((unsigned short)(w & 0xffffu)); }

__device__ __forceinline__ void ll_st(uint32_t* p, uint32_t w) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(w) : "memory");
}

__device__ __forceinline__ void ll_st2(uint32_t* p, uint32_t w0, uint32_t w1) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(w0), "r"(w1) : "memory");
}

// One more failed poll: gives up after the limit, or as soon as somebody else has given up.
__device__ __forceinline__ bool ll_give_up(LLWait& w, unsigned& spins) {
    if (++spins > LL_SPIN_LIMIT) {
        atomicOr(w.flag, FLAG_LL_TIMEOUT);
        w.dead = true;
        return true;
    }
    if ((spins & 1023u) == 0) {
        int f;
        asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(w.flag) : "memory");
        if (f & FLAG_LL_TIMEOUT) {
            w.dead = true;
            return true;
        }
    }
    return false;
}

__device__ __forceinline__ uint4 ll_raw4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ bool ll_ok4(const uint4& v, uint32_t tag) {
    return (v.x >> 16) == tag && (v.y >> 16) == tag && (v.z >> 16) == tag && (v.w >> 16) == tag;
}

__device__ __forceinline__ uint32_t ll_ld1(const uint32_t* p, uint32_t tag, LLWait& w) {
    uint32_t v;
    unsigned spins = 0;
    for (;;) {
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
        if ((v >> 16) == tag || w.dead) break;
        if (ll_give_up(w, spins)) break;
        __nanosleep(spins < 4 ? 32 : 256);
    }
    return v;
}

__device__ __forceinline__ uint4 ll_pack8(const uint4& a, const uint4& b) {
    uint4 r;
    r.x = (a.x & 0xffffu) | (a.y << 16);
    r.y = (a.z & 0xffffu) | (a.w << 16);
    r.z = (b.x & 0xffffu) | (b.y << 16);
    r.w = (b.z & 0xffffu) | (b.w << 16);
    return r;
}

// N groups of 8 consecutive elements (32 bytes of words each, 32-byte aligned) as packed bf16, group i
// expected with tag[i]; groups with on[i] == false are skipped.  All 2N loads of a round are in flight
// together and the round is repeated until every word carries its tag: one L2 round trip when the
// producers are done, whatever N.
template <int N>
__device__ __forceinline__ void ll_ld8n(const uint32_t* (&p)[N], const uint32_t (&tag)[N], const bool (&on)[N],
                                        uint4 (&out)[N], LLWait& w) {
    uint4 a[N], b[N];
    bool need[N];
#pragma unroll
    for (int i = 0; i < N; ++i) need[i] = on[i];
    unsigned spins = 0;
    for (;;) {
        // only the groups that are not complete yet are fetched again: the waiting CTAs must not
        // flood the L2 that the producers still need for their weights
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (need[i]) {
                a[i] = ll_raw4(p[i]);
                b[i] = ll_raw4(p[i] + 4);
            }
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (need[i]) {
                need[i] = !(ll_ok4(a[i], tag[i]) && ll_ok4(b[i], tag[i]));
                ok = ok && !need[i];
            }
        if (ok || w.dead) break;
        if (ll_give_up(w, spins)) break;
        __nanosleep(spins < 4 ? 32 : 256);
    }
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = on[i] ? ll_pack8(a[i], b[i]) : make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ uint4 ll_ld8(const uint32_t* p, uint32_t tag, LLWait& w) {
    const uint32_t* pp[1] = {p};
    const uint32_t tt[1] = {tag};
    const bool on[1] = {true};
    uint4 out[1];
    ll_ld8n<1>(pp, tt, on, out, w);
    return out[0];
}

// ---------------------------------------------------------------------------------------------
// Staging functors over tagged rows (the arithmetic is that of StageNorm / StageCopy / StageRqAttn).
// ---------------------------------------------------------------------------------------------
struct TStageNorm {
    const uint32_t* x;  // row r of the product lives at x + (r*row_mul + row_add)*K
    uint32_t tag;
    const bf16* w;
    float eps;
    int row_mul, row_add;
    LLWait* wt;
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr) const {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int rr = warp; rr < nr; rr += (int)(blockDim.x >> 5)) {
            const uint32_t* xr = x + ((size_t)(r0 + rr) * row_mul + row_add) * K;
            constexpr int IT = (K + 255) / 256;
            float v[IT][8];
            float ss = 0.f;
            {
                const uint32_t* pp[IT];
                uint32_t tt[IT];
                bool on[IT];
                uint4 raw[IT];
#pragma unroll
                for (int it = 0; it < IT; ++it) {
                    const int k = it * 256 + lane * 8;
                    on[it] = k < K;
                    pp[it] = xr + (on[it] ? k : 0);
                    tt[it] = tag;
                }
                ll_ld8n<IT>(pp, tt, on, raw, *wt);
#pragma unroll
                for (int it = 0; it < IT; ++it) {
                    if (on[it]) {
                        unpack8(raw[it], v[it]);
#pragma unroll
                        for (int j = 0; j < 8; ++j) ss = fmaf(v[it][j], v[it][j], ss);
                    }
                }
            }
            ss = warp_sum(ss);
            const float rinv = rsqrtf(ss / (float)K + eps);
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int k = it * 256 + lane * 8;
                if (k < K) {
                    float wf[8], o[8];
                    unpack8(__ldg(reinterpret_cast<const uint4*>(w + k)), wf);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = rbf(v[it][j] * rinv) * wf[j];
                    *reinterpret_cast<uint4*>(Xs + rr * K + k) = pack8(o);
                }
            }
        }
    }
};

struct TStageCopy {
    const uint32_t* x;  // (M, K) words
    uint32_t tag;
    LLWait* wt;
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr) const {
        const uint32_t* src = x + (size_t)r0 * K;
        uint4* dst = reinterpret_cast<uint4*>(Xs);
        const int n = nr * (K / 8), step = (int)blockDim.x;
        for (int i0 = threadIdx.x; i0 < n; i0 += 4 * step) {
            const uint32_t* pp[4];
            uint32_t tt[4];
            bool on[4];
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * step;
                on[u] = i < n;
                pp[u] = src + (size_t)(on[u] ? i : 0) * 8;
                tt[u] = tag;
            }
            ll_ld8n<4>(pp, tt, on, raw, *wt);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (on[u]) dst[i0 + u * step] = raw[u];
        }
    }
};

struct TStageRqAttn {
    const uint32_t* q;  // (M, H*64) words
    uint32_t tag_q;
    const uint32_t* kc;  // (R, Qpos, H*64) words, this layer
    const uint32_t* vc;
    const uint32_t* kv_tag;  // [Qpos] in shared memory: tag of each position of this layer
    int H, Qpos, rows_per_b, pos_base;
    LLWait* wt;
    template <int K>
    __device__ __forceinline__ void stage(bf16* Xs, int r0, int nr) const {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int s = lane & 7, g = lane >> 3;
        for (int rr = 0; rr < nr; ++rr) {
            const int r = r0 + rr;
            const int b = r / rows_per_b, pos = pos_base + r % rows_per_b;
            for (int h = warp; h < H; h += (int)(blockDim.x >> 5)) {
                // q and the first 8 positions in one poll, positions 8..15 (later passes) in a second one
                float qf[8];
                float m = NEG_BIG, l = 0.f, acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half * 8 <= pos) {  // the whole warp takes the same halves
                        const uint32_t* pp[5];
                        uint32_t tt[5];
                        bool on[5];
                        uint4 raw[5];
                        pp[0] = q + (size_t)r * K + h * HD + s * 8;
                        tt[0] = tag_q;
                        on[0] = half == 0;
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int t = half * 8 + u * 4 + g;
                            const bool ok = t <= pos;
                            const int tt_ = ok ? t : 0;
                            const size_t off = ((size_t)b * Qpos + tt_) * K + h * HD + s * 8;
                            pp[1 + 2 * u] = kc + off;
                            pp[2 + 2 * u] = vc + off;
                            tt[1 + 2 * u] = tt[2 + 2 * u] = kv_tag[tt_];
                            on[1 + 2 * u] = on[2 + 2 * u] = ok;
                        }
                        ll_ld8n<5>(pp, tt, on, raw, *wt);
                        if (half == 0) unpack8(raw[0], qf);
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            if (half * 8 + u * 4 <= pos) {
                                const int t = half * 8 + u * 4 + g;
                                const bool ok = t <= pos;
                                float kf[8], vf[8];
                                unpack8(raw[1 + 2 * u], kf);
                                unpack8(raw[2 + 2 * u], vf);
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

// ---------------------------------------------------------------------------------------------
// Epilogue functors writing tagged words (the arithmetic is that of EpiQkv / EpiResidual / ...).
// ---------------------------------------------------------------------------------------------
struct TEpiQkv {
    const bf16* W;
    int K;
    uint32_t* q_out;  // (M, q_cols) words
    int q_cols, kv_cols;
    // backbone: new k | v of row r at kv_new + r * 2 * kv_cols, and the bf16 cache for the frames to come
    uint32_t* kv_new;
    bf16* k_cache;
    bf16* v_cache;
    const int* s_slot;  // shared memory, backbone only
    const int* s_pos;
    int max_seq;
    const bf16* rope;
    // depth transformer (kv_new == NULL): tagged cache (R, Qpos, kv_cols)
    uint32_t* kc_t;
    uint32_t* vc_t;
    int rows_per_b, pos_base;
    uint32_t tag;
    static constexpr int NC = 2;
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[2]) const {
        wr[0] = W + (size_t)(2 * item) * K;
        wr[1] = wr[0] + K;
    }
    __device__ __forceinline__ uint32_t pre(int item, int r0, int nr, int lane) const {
        return 0u;
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane, const float (&acc)[2][RT], uint32_t pre) const {
        if (lane >= nr) return;
        const int r = r0 + lane;
        const int n = 2 * item;
        float t0 = rbf(pick<RT>(acc[0], lane)), t1 = rbf(pick<RT>(acc[1], lane));
        int slot, pos;
        if (kv_new) {
            slot = s_slot[r];
            pos = s_pos[r];
        } else {
            slot = r / rows_per_b;
            pos = pos_base + r % rows_per_b;
        }
        if (rope && n < q_cols + kv_cols) {
            const int dd = n & (HD - 1);
            const bf16* f = rope + ((size_t)pos * HD + dd) * 2;
            const float c0 = bf2f(f[0]), s0 = bf2f(f[1]), c1 = bf2f(f[2]), s1 = bf2f(f[3]);
            const float o0 = rbf(rbf(t0 * c0) + rbf((-t1) * s0));
            const float o1 = rbf(rbf(t1 * c1) + rbf(t0 * s1));
            t0 = o0;
            t1 = o1;
        }
        const bf16 b0 = f2bf(t0), b1 = f2bf(t1);
        const uint32_t w0 = ll_word(b0, tag), w1 = ll_word(b1, tag);
        if (n < q_cols) {
            ll_st2(q_out + (size_t)r * q_cols + n, w0, w1);
        } else if (kv_new) {
            const int col = n - q_cols;  // 0 .. 2*kv_cols: k then v
            ll_st2(kv_new + (size_t)r * 2 * kv_cols + col, w0, w1);
            __nv_bfloat162 pr;
            pr.x = b0;
            pr.y = b1;
            bf16* cache = col < kv_cols ? k_cache : v_cache;
            *reinterpret_cast<__nv_bfloat162*>(cache + ((size_t)slot * max_seq + pos) * kv_cols + (col % kv_cols)) = pr;
        } else if (n < q_cols + kv_cols) {
            ll_st2(kc_t + ((size_t)slot * max_seq + pos) * kv_cols + (n - q_cols), w0, w1);
        } else {
            ll_st2(vc_t + ((size_t)slot * max_seq + pos) * kv_cols + (n - q_cols - kv_cols), w0, w1);
        }
    }
};

struct TEpiResidual {
    const bf16* W;
    int K;
    uint32_t* x;  // (M, N) words, updated in place
    int N;
    bf16* tap;
    uint32_t tag_old, tag_new;
    LLWait* wt;
    static constexpr int NC = 1;
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[1]) const { wr[0] = W + (size_t)item * K; }
    __device__ __forceinline__ uint32_t pre(int item, int r0, int nr, int lane) const {
        // the word this lane will add to, requested before the dot products hide its latency
        if (lane >= nr) return 0u;
        uint32_t v;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(x + (size_t)(r0 + lane) * N + item) : "memory");
        return v;
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane, const float (&acc)[1][RT], uint32_t pre) const {
        if (lane >= nr) return;
        const size_t idx = (size_t)(r0 + lane) * N + item;
        if ((pre >> 16) != tag_old) pre = ll_ld1(x + idx, tag_old, *wt);
        const bf16 old = ll_val(pre);
        const bf16 o = f2bf(bf2f(old) + rbf(pick<RT>(acc[0], lane)));
        ll_st(x + idx, ll_word(o, tag_new));
        if (tap) tap[idx] = o;
    }
};

struct TEpiSwiGLU {
    const bf16* W1;
    const bf16* W3;
    int K;
    uint32_t* act;  // (M, F) words
    int F;
    uint32_t tag;
    static constexpr int NC = 2;
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[2]) const {
        wr[0] = W1 + (size_t)item * K;
        wr[1] = W3 + (size_t)item * K;
    }
    __device__ __forceinline__ uint32_t pre(int item, int r0, int nr, int lane) const {
        return 0u;
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane, const float (&acc)[2][RT], uint32_t pre) const {
        if (lane >= nr) return;
        const float a = rbf(pick<RT>(acc[0], lane)), g = rbf(pick<RT>(acc[1], lane));
        const float s = rbf(a / (1.0f + expf(-a)));
        ll_st(act + (size_t)(r0 + lane) * F + item, ll_word(f2bf(s * g), tag));
    }
};

struct TEpiLogits {
    const bf16* W;  // (n_main, K)
    int K, n_main;
    uint32_t* out;  // rows of out_stride words; word n_main of a row is the extra output
    int out_stride;
    const bf16* W_extra;
    const bf16* b_extra;
    bf16* tap;
    int tap_stride;
    uint32_t tag;
    static constexpr int NC = 1;
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[1]) const {
        wr[0] = item < n_main ? W + (size_t)item * K : W_extra;
    }
    __device__ __forceinline__ uint32_t pre(int item, int r0, int nr, int lane) const {
        return 0u;
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane, const float (&acc)[1][RT], uint32_t pre) const {
        if (lane >= nr) return;
        const int r = r0 + lane;
        const float v = pick<RT>(acc[0], lane);
        if (item < n_main) {
            const bf16 o = f2bf(v);
            ll_st(out + (size_t)r * out_stride + item, ll_word(o, tag));
            if (tap) tap[(size_t)r * tap_stride + item] = o;
        } else {
            ll_st(out + (size_t)r * out_stride + n_main, ll_word(f2bf(v + bf2f(b_extra[0])), tag));
        }
    }
};

struct TEpiProjPos {
    const bf16* W;
    int K;
    const bf16* pos_emb;
    uint32_t* out;  // row of stream b is b*row_mul, rd words each
    int rd, row_mul;
    uint32_t tag;
    static constexpr int NC = 1;
    __device__ __forceinline__ void rows(int item, const bf16* (&wr)[1]) const { wr[0] = W + (size_t)item * K; }
    __device__ __forceinline__ uint32_t pre(int item, int r0, int nr, int lane) const {
        return 0u;
    }
    template <int RT>
    __device__ __forceinline__ void store(int item, int r0, int nr, int lane, const float (&acc)[1][RT], uint32_t pre) const {
        if (lane >= nr) return;
        const int b = r0 + lane;
        ll_st(out + (size_t)b * row_mul * rd + item, ll_word(f2bf(rbf(pick<RT>(acc[0], lane)) + bf2f(pos_emb[item])), tag));
    }
};

// ---------------------------------------------------------------------------------------------
// Backbone attention: attn_unit of the per-phase kernels with q, the key/value of the current
// position and the output as tagged words; earlier positions come from the bf16 cache.
// ---------------------------------------------------------------------------------------------
struct LLAttnArgs {
    const uint32_t* q;       // (R, Hq*64) words
    const uint32_t* kv_new;  // (R, 2*Hkv*64) words
    uint32_t tag_in;
    const bf16* kc;
    const bf16* vc;
    const int* s_slot;
    const int* s_pos;
    float* part;
    int32_t* counters;
    uint32_t* out;  // (R, Hq*64) words
    uint32_t tag_out;
    int Hq, Hkv, max_seq, S;
    LLWait* wt;
};

__device__ __forceinline__ void ll_attn_unit(const LLAttnArgs& a, int sp, int kvh, int r, int tid, AttnSmem& S_,
                                             int bar_id) {
    const int pos = a.s_pos[r];
    const int len = pos + 1;
    const int nsplit = (len + ATT_SPLIT - 1) / ATT_SPLIT;
    if (sp >= nsplit) return;
    const int slot = a.s_slot[r];
    const int warp = tid >> 5, lane = tid & 31;
    const int s = lane & 7, g = lane >> 3;
    const int G = a.Hq / a.Hkv;
    const int t_begin = sp * ATT_SPLIT, t_end = min(len, t_begin + ATT_SPLIT);
    const size_t pos_stride = (size_t)a.Hkv * HD;
    const bf16* kb = a.kc + (size_t)slot * a.max_seq * pos_stride + kvh * HD + s * 8;
    const bf16* vb = a.vc + (size_t)slot * a.max_seq * pos_stride + kvh * HD + s * 8;

    uint4 kr[ATT_ITERS], vr[ATT_ITERS];
#pragma unroll
    for (int it = 0; it < ATT_ITERS; ++it) {
        const int t = t_begin + it * 16 + warp * 4 + g;
        if (t < t_end && t != pos) {
            kr[it] = ldg_stream(kb + (size_t)t * pos_stride);
            vr[it] = ldg_stream(vb + (size_t)t * pos_stride);
        } else {
            kr[it] = make_uint4(0, 0, 0, 0);
            vr[it] = make_uint4(0, 0, 0, 0);
        }
    }
    float (&sm)[4][2][8][10] = S_.sm;
    int& s_last = S_.s_last;
    // q of both heads and, where this lane's key is the current position, its k and v (they come from
    // the exchange buffer: the cache line may not have landed yet) in one poll
    float qf[2][8];
    {
        bool mine = false;
#pragma unroll
        for (int it = 0; it < ATT_ITERS; ++it) mine = mine || (t_begin + it * 16 + warp * 4 + g == pos);
        const uint32_t* kn = a.kv_new + (size_t)r * 2 * pos_stride + kvh * HD + s * 8;
        const uint32_t* pq[2] = {a.q + (size_t)r * a.Hq * HD + (kvh * G) * HD + s * 8,
                                 a.q + (size_t)r * a.Hq * HD + (kvh * G + (G > 1 ? 1 : 0)) * HD + s * 8};
        const uint32_t* pk[2] = {kn, kn + pos_stride};
        const uint32_t tt[2] = {a.tag_in, a.tag_in};
        const bool on_q[2] = {true, true}, on_k[2] = {mine, mine};
        uint4 rq[2], rk[2];
        ll_ld8n<2>(pq, tt, on_q, rq, *a.wt);
        ll_ld8n<2>(pk, tt, on_k, rk, *a.wt);
        unpack8(rq[0], qf[0]);
        unpack8(rq[1], qf[1]);
#pragma unroll
        for (int it = 0; it < ATT_ITERS; ++it) {
            if (t_begin + it * 16 + warp * 4 + g == pos) {
                kr[it] = rk[0];
                vr[it] = rk[1];
            }
        }
    }
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
    bar_named(bar_id, ATT_THREADS);
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
    uint32_t* outp = a.out + (size_t)r * a.Hq * HD + hq * HD + dim;
    if (nsplit == 1) {
        if (head_ok) ll_st(outp, ll_word(f2bf(O_ / L_), a.tag_out));
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
    bar_named(bar_id, ATT_THREADS);  // every thread's partial stores precede thread 0's release below
    if (tid == 0) {
        int old;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(a.counters + r * a.Hkv + kvh) : "memory");
        s_last = (old == nsplit - 1);
    }
    bar_named(bar_id, ATT_THREADS);
    if (!s_last) return;
    if (head_ok) {
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
        ll_st(outp, ll_word(f2bf(Os / Ls), a.tag_out));
    }
    if (tid == 0) a.counters[r * a.Hkv + kvh] = 0;
}

// Depth token for position p as tagged words: code_emb[(p-1)*CS + code] + pos_emb[p].
__device__ __forceinline__ void ll_embed_row(int code, const bf16* code_emb, const bf16* pos_emb, uint32_t* out_row,
                                             int rd, int CS, int p, int tid, uint32_t tag) {
    const bf16* e = code_emb + ((size_t)(p - 1) * CS + code) * rd;
    const bf16* pe = pos_emb + (size_t)p * rd;
    for (int k = tid * 2; k < rd; k += SAMPLE_THREADS * 2) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(e + k);
        const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(pe + k);
        ll_st2(out_row + k, ll_word(f2bf(bf2f(a.x) + bf2f(c.x)), tag), ll_word(f2bf(bf2f(a.y) + bf2f(c.y)), tag));
    }
}

// Row r of a tagged logits buffer -> plain bf16 row (thread t copies the 8 values it samples from).
__device__ __forceinline__ void ll_fetch_logits(const uint32_t* src, bf16* dst, int CS, int tid, uint32_t tag, LLWait& w) {
    for (int i = tid; i < CS / 8; i += SAMPLE_THREADS)
        *reinterpret_cast<uint4*>(dst + (size_t)i * 8) = ll_ld8(src + (size_t)i * 8, tag, w);
}

// Profiling aid: CTA 0 appends device-clock stamps to the trace region (three per phase).
struct LLTrace {
    unsigned long long* buf;  // NULL when tracing is off
    unsigned n;
};

__device__ __forceinline__ void ll_stamp(LLTrace& t) {
    if (t.buf && blockIdx.x == 0 && threadIdx.x == 0 && t.n < 2 * TRACE_MAX) {
        t.buf[1 + t.n] = globaltimer_ns();
        ++t.n;
        t.buf[0] = (t.n + 1) / 2;
    }
}

// A phase of matrix-vector products (gemv_phase of the barrier version with two changes).  No grid
// barrier separates the phases here, so the CTA itself makes sure that every warp is done with the
// staged tile of the previous phase before it is refilled; and the epilogue may request what it needs
// from global memory before the dot products.
template <int K, int RT, class Stage, class Epi>
__device__ __forceinline__ void ll_phase(const Stage& st, const Epi& ep, int M, int n_items, bf16* Xs,
                                         WPref<K, Epi>& p, LLTrace& tr) {
    constexpr int NC = Epi::NC;
    constexpr int IT = (K + 255) / 256;
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * PF_WARPS + (threadIdx.x >> 5), tw = gridDim.x * PF_WARPS;
    for (int r0 = 0; r0 < M; r0 += RT) {
        const int nr = min(RT, M - r0);
        __syncthreads();
        ll_stamp(tr);
        st.template stage<K>(Xs, r0, nr);
        __syncthreads();
        ll_stamp(tr);
        int nth = 0;
        for (int item = gw; item < n_items; item += tw, ++nth) {
            if (nth > 0 || (r0 > 0 && n_items > tw)) wload<K, Epi>(ep, item, p);
            uint32_t pre = ep.pre(item, r0, nr, lane);
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
            ep.template store<RT>(item, r0, nr, lane, acc, pre);
        }
        ll_stamp(tr);
    }
}

template <int RT, int RQF>
__global__ void __launch_bounds__(PF_THREADS, 1) k_frame_ll(LLArgs la) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Xs = reinterpret_cast<bf16*>(smem_raw);
    __shared__ AttnSmem att_sm[PF_ATT_GROUPS];
    __shared__ SampleSmem samp_sm;
    __shared__ int s_slot[LL_MAXB], s_pos[LL_MAXB];
    __shared__ uint32_t kv_tag[LLLayout::RL][LLLayout::Q];
    constexpr int D = 1024, F = 3072, RD = 512;
    typedef LLLayout LY;
    const FrameArgs& a = la.fa;
    const DevModel& m = *a.m;
    const FrameBufs& b = a.b;
    const int B = a.B, cta = blockIdx.x, tid = threadIdx.x;
    const int qc = a.n_heads * HD, kvc = a.n_kv_heads * HD;
    const int Qn = a.n_codebooks;
    uint32_t* const TX = la.bufs + LY::X;
    uint32_t* const TQ = la.bufs + LY::QO;
    uint32_t* const TKV = la.bufs + LY::KV;
    uint32_t* const TATT = la.bufs + LY::ATT;
    uint32_t* const TACT = la.bufs + LY::ACT;
    uint32_t* const THID = la.bufs + LY::HID;
    uint32_t* const TCB0 = la.bufs + LY::CB0;
    uint32_t* const TRX2 = la.bufs + LY::RX2;
    uint32_t* const TRX = la.bufs + LY::RX;
    uint32_t* const TRQ = la.bufs + LY::RQ;
    uint32_t* const TRACT = la.bufs + LY::RACT;
    uint32_t* const TRLOG = la.bufs + LY::RLOG;
    uint32_t* const TRK = la.bufs + LY::RK;
    uint32_t* const TRV = la.bufs + LY::RV;
    LLWait wt{b.flag, false};
    LLTrace tr{b.trace, 0u};

    // ---- shape guard: words older than one launch may carry any tag -------------------------------
    uint32_t g = la.state[0];
    const uint32_t shape = (uint32_t)B | ((uint32_t)Qn << 8) | 0x80000000u;
    const bool reshape = la.state[1] != shape;
    if (reshape) {
        uint4* p4 = reinterpret_cast<uint4*>(la.bufs);
        for (size_t i = (size_t)cta * PF_THREADS + tid; i < LY::END / 4; i += (size_t)gridDim.x * PF_THREADS)
            p4[i] = make_uint4(0, 0, 0, 0);
        __threadfence();
        GridBarrier bar{la.state + 2, 0u, gridDim.x, b.flag, false, nullptr, 0u};
        bar.sync();
    }

    // ---- rows: slot and position of every stream (each CTA for itself; seq_lens moves only at the end)
    if (tid < B) {
        int slot = a.slots[tid];
        if (slot < 0 || slot >= a.n_slots) {
            atomicOr(b.flag, FLAG_BAD_SLOT);
            slot = a.n_slots - 1;
        }
        int pos = m.seq_lens[slot];
        if (pos < 0 || pos >= a.max_seq) {
            atomicOr(b.flag, FLAG_BAD_POS);
            pos = pos < 0 ? 0 : a.max_seq - 1;
        }
        s_slot[tid] = slot;
        s_pos[tid] = pos;
        if (cta == 0) {
            b.row_slot[tid] = slot;
            b.row_pos[tid] = pos;
        }
    }
    __syncthreads();

    // ---- embed: CTA r gathers and sums the 16 table rows of stream r -----------------------------
    uint32_t x_tag = ll_tag(++g);
    if (cta < B) {
        const int r = cta;
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
#pragma unroll
            for (int j = 0; j < 8; j += 2)
                ll_st2(TX + (size_t)r * D + k + j, ll_word(f2bf(acc[j]), x_tag), ll_word(f2bf(acc[j + 1]), x_tag));
        }
    }

    for (int li = 0; li < a.n_layers; ++li) {
        const uint32_t t_qkv = ll_tag(++g);
        {
            TEpiQkv eq{static_cast<const bf16*>(m.w.wqkv[li]), D, TQ, qc, kvc, TKV,
                       static_cast<bf16*>(m.k[li]), static_cast<bf16*>(m.v[li]), s_slot, s_pos, a.max_seq, m.rope,
                       nullptr, nullptr, 1, 0, t_qkv};
            WPref<D, TEpiQkv> wq;
            wprefetch<D>(eq, (qc + 2 * kvc) / 2, wq);
            TStageNorm sn{TX, x_tag, static_cast<const bf16*>(m.w.attn_norm[li]), a.norm_eps, 1, 0, &wt};
            ll_phase<D, RT>(sn, eq, B, (qc + 2 * kvc) / 2, Xs, wq, tr);
        }
        const uint32_t t_att = ll_tag(++g);
        TEpiResidual eo{static_cast<const bf16*>(m.w.out_proj[li]), D, TX, D, nullptr, x_tag, 0u, &wt};
        WPref<D, TEpiResidual> wo;
        wprefetch<D>(eo, D, wo);
        {   // attention: a group of 128 threads per (split, kv head, row) unit
            LLAttnArgs aa{TQ, TKV, t_qkv, static_cast<const bf16*>(m.k[li]), static_cast<const bf16*>(m.v[li]),
                          s_slot, s_pos, b.part, b.counters, TATT, t_att, a.n_heads, a.n_kv_heads, a.max_seq, a.S, &wt};
            const int group = tid / ATT_THREADS, gt = tid % ATT_THREADS;
            const int units = a.S * a.n_kv_heads * B;
            for (int u = cta * PF_ATT_GROUPS + group; u < units; u += gridDim.x * PF_ATT_GROUPS) {
                bar_named(1 + group, ATT_THREADS);
                ll_attn_unit(aa, u % a.S, (u / a.S) % a.n_kv_heads, u / (a.S * a.n_kv_heads), gt, att_sm[group], 1 + group);
            }
        }
        {
            eo.tag_new = ll_tag(++g);
            TStageCopy sc{TATT, t_att, &wt};
            ll_phase<D, RT>(sc, eo, B, D, Xs, wo, tr);
            x_tag = eo.tag_new;
        }
        const uint32_t t_act = ll_tag(++g);
        {
            TEpiSwiGLU eg{static_cast<const bf16*>(m.w.w1[li]), static_cast<const bf16*>(m.w.w3[li]), D, TACT, F, t_act};
            WPref<D, TEpiSwiGLU> wg;
            wprefetch<D>(eg, F, wg);
            TStageNorm sm{TX, x_tag, static_cast<const bf16*>(m.w.mlp_norm[li]), a.norm_eps, 1, 0, &wt};
            ll_phase<D, RT>(sm, eg, B, F, Xs, wg, tr);
        }
        {
            bf16* tap = a.tap_layers ? a.tap_layers + (size_t)li * a.max_rows * D : nullptr;
            TEpiResidual ew{static_cast<const bf16*>(m.w.w2[li]), F, TX, D, tap, x_tag, ll_tag(++g), &wt};
            WPref<F, TEpiResidual> ww;
            wprefetch<F>(ew, D, ww);
            TStageCopy sa{TACT, t_act, &wt};
            ll_phase<F, RT>(sa, ew, B, D, Xs, ww, tr);
            x_tag = ew.tag_new;
        }
    }
    // ---- final norm + codec_head + eos_head --------------------------------------------------------
    const uint32_t t_head = ll_tag(++g);
    {
        TEpiLogits el{static_cast<const bf16*>(m.w.codec_head), D, a.CS, TCB0, (int)LY::CB0_STRIDE,
                      static_cast<const bf16*>(m.w.eos_w), static_cast<const bf16*>(m.w.eos_b), nullptr, 0, t_head};
        WPref<D, TEpiLogits> wh;
        wprefetch<D>(el, a.CS + 1, wh);
        TStageNorm sf{TX, x_tag, static_cast<const bf16*>(m.w.final_norm), a.norm_eps, 1, 0, &wt};
        ll_phase<D, RT>(sf, el, B, a.CS + 1, Xs, wh, tr);
        if (cta == 0) {  // B <= RT: the staged tile is the final-norm output of every row
            for (int i = tid; i < B * (D / 8); i += PF_THREADS) {
                const uint4 v = reinterpret_cast<const uint4*>(Xs)[i];
                reinterpret_cast<uint4*>(a.hidden_out)[i] = v;
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    ll_st2(THID + (size_t)i * 8 + 2 * j, (w[j] & 0xffffu) | (t_head << 16), (w[j] >> 16) | (t_head << 16));
            }
            if (tid < B) {
                const int inc = a.seq_inc ? a.seq_inc[tid] : 1;
                if (inc) m.seq_lens[s_slot[tid]] += inc;
            }
        }
    }

    // ---- depth step ------------------------------------------------------------------------------
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
    uint32_t rx_tag = ll_tag(++g);  // depth positions 0 (projection of the hidden state) and 1 (cb0 token)
    {
        TEpiProjPos ep{static_cast<const bf16*>(m.w.rq_backbone_proj), D, pos_emb, TRX2, RD, 2, rx_tag};
        WPref<D, TEpiProjPos> wp;
        wprefetch<D>(ep, RD, wp);
        TStageCopy sh{THID, t_head, &wt};
        ll_phase<D, RT>(sh, ep, B, RD, Xs, wp, tr);
        if (cta < B && tid < SAMPLE_THREADS) {  // cb0, then depth position 1 from it
            ll_fetch_logits(TCB0 + (size_t)cta * LY::CB0_STRIDE, a.cb0_out + (size_t)cta * a.CS, a.CS, tid, t_head, wt);
            if (tid == 0) a.eos_out[cta] = ll_val(ll_ld1(TCB0 + (size_t)cta * LY::CB0_STRIDE + a.CS, t_head, wt));
            bar_named(5, SAMPLE_THREADS);
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
            ll_embed_row(code, code_emb, pos_emb, TRX2 + ((size_t)2 * cta + 1) * RD, RD, a.CS, 1, tid, rx_tag);
        }
    }
    sa.eos_logit = nullptr;
    sa.eos_prob = nullptr;
    sa.first_frame = 0;
    sa.zero_from = 0;

    const bf16* head = static_cast<const bf16*>(m.w.rq_head);
    const size_t layer_kv = (size_t)LL_MAXB * LY::Q * RD;
    for (int i = 0; i < Qn - 1 || i == 0; ++i) {
        // ---- the depth layers: positions 0 and 1 together (2 rows per stream), then one position a pass
        if (i == 0 || i < Qn - 1) {
            const int rows_per_b = i == 0 ? 2 : 1, pos_base = i == 0 ? 0 : i + 1, M = i == 0 ? 2 * B : B;
            uint32_t* x = i == 0 ? TRX2 : TRX;
            for (int li = 0; li < a.rq_n_layers; ++li) {
                uint32_t* kc = TRK + li * layer_kv;
                uint32_t* vc = TRV + li * layer_kv;
                const uint32_t t_q = ll_tag(++g);
                __syncthreads();  // the previous readers of kv_tag are done
                if (tid < rows_per_b) kv_tag[li][pos_base + tid] = t_q;
                {
                    TEpiQkv eq{static_cast<const bf16*>(m.w.rq_wqkv[li]), RD, TRQ, RD, RD, nullptr, nullptr, nullptr,
                               nullptr, nullptr, (int)LY::Q, nullptr, kc, vc, rows_per_b, pos_base, t_q};
                    WPref<RD, TEpiQkv> wq;
                    wprefetch<RD>(eq, 3 * RD / 2, wq);
                    TStageNorm sn{x, rx_tag, static_cast<const bf16*>(m.w.rq_attn_norm[li]), a.rq_norm_eps, 1, 0, &wt};
                    ll_phase<RD, RT>(sn, eq, M, 3 * RD / 2, Xs, wq, tr);
                }
                {
                    TEpiResidual eo{static_cast<const bf16*>(m.w.rq_out_proj[li]), RD, x, RD, nullptr, rx_tag, ll_tag(++g), &wt};
                    WPref<RD, TEpiResidual> wo;
                    wprefetch<RD>(eo, RD, wo);
                    TStageRqAttn st{TRQ, t_q, kc, vc, kv_tag[li], a.rq_n_heads, (int)LY::Q, rows_per_b, pos_base, &wt};
                    ll_phase<RD, RT>(st, eo, M, RD, Xs, wo, tr);
                    rx_tag = eo.tag_new;
                }
                const uint32_t t_act = ll_tag(++g);
                {
                    TEpiSwiGLU eg{static_cast<const bf16*>(m.w.rq_w1[li]), static_cast<const bf16*>(m.w.rq_w3[li]), RD,
                                  TRACT, RQF, t_act};
                    WPref<RD, TEpiSwiGLU> wg;
                    wprefetch<RD>(eg, RQF, wg);
                    TStageNorm sm{x, rx_tag, static_cast<const bf16*>(m.w.rq_mlp_norm[li]), a.rq_norm_eps, 1, 0, &wt};
                    ll_phase<RD, RT>(sm, eg, M, RQF, Xs, wg, tr);
                }
                {
                    TEpiResidual ew{static_cast<const bf16*>(m.w.rq_w2[li]), RQF, x, RD, nullptr, rx_tag, ll_tag(++g), &wt};
                    WPref<RQF, TEpiResidual> ww;
                    wprefetch<RQF>(ew, RD, ww);
                    TStageCopy sc{TRACT, t_act, &wt};
                    ll_phase<RQF, RT>(sc, ew, M, RD, Xs, ww, tr);
                    rx_tag = ew.tag_new;
                }
            }
        }
        if (i >= Qn - 1) break;  // a single codebook: the layers above only fill the depth KV
        // ---- head i -> code i+1 -------------------------------------------------------------------
        const uint32_t t_log = ll_tag(++g);
        {
            TEpiLogits el{head + (size_t)i * a.CS * RD, RD, a.CS, TRLOG, a.CS, nullptr, nullptr,
                          a.tap_rq ? a.tap_rq + (size_t)i * a.CS : nullptr, (a.Q - 1) * a.CS, t_log};
            WPref<RD, TEpiLogits> wh;
            wprefetch<RD>(el, a.CS, wh);
            TStageNorm sn{i == 0 ? TRX2 : TRX, rx_tag, static_cast<const bf16*>(m.w.rq_norm), a.rq_norm_eps,
                          i == 0 ? 2 : 1, i == 0 ? 1 : 0, &wt};
            ll_phase<RD, RT>(sn, el, B, a.CS, Xs, wh, tr);
        }
        const uint32_t t_tok = ll_tag(++g);
        if (cta < B && tid < SAMPLE_THREADS) {
            ll_fetch_logits(TRLOG + (size_t)cta * a.CS, b.rq_logits + (size_t)cta * a.CS, a.CS, tid, t_log, wt);
            bar_named(5, SAMPLE_THREADS);
            sa.logits = b.rq_logits;
            sa.stride = a.CS;
            sa.codebook = i + 1;
            sa.out_col = i + 1;
            sa.bump_frame = (i == Qn - 2);
            const int code = sample_row(sa, cta, tid, samp_sm, 5);
            if (i + 1 < Qn - 1) ll_embed_row(code, code_emb, pos_emb, TRX + (size_t)cta * RD, RD, a.CS, i + 2, tid, t_tok);
        }
        rx_tag = t_tok;
    }

    if (cta == 0 && tid == 0) {
        la.state[0] = g;
        la.state[1] = shape;
        if (reshape) la.state[2] = 0;
    }
}

typedef void (*LLKernel)(LLArgs);

template <int RQF>
static LLKernel ll_kernel_for(int rt) {
    switch (rt) {
        case 1: return k_frame_ll<1, RQF>;
        case 2: return k_frame_ll<2, RQF>;
        default: return k_frame_ll<4, RQF>;
    }
}

int launch_frame_ll(const LLArgs& a, int rq_ffn, int num_sms, bool cooperative, cudaStream_t s) {
    const int B = a.fa.B;
    const int rt = B <= 1 ? 1 : B <= 2 ? 2 : 4;
    LLKernel kern = rq_ffn == 1408 ? ll_kernel_for<1408>(rt) : ll_kernel_for<1536>(rt);
    const size_t smem = (size_t)rt * 3072 * sizeof(bf16);
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms);
    cfg.blockDim = dim3(PF_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cooperative ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace vuib
