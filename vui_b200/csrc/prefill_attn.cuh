// Causal attention of a PREFILL call on the tensor cores: query tile x key tile.
//
// The decode attention kernel gives every row a grid slice of its own; a prefill of thousands of rows
// pays for that in launches of tens of thousands of CTAs per layer.  Here the rows of a call are cut
// into tiles of up to 64 consecutive positions of one slot (k_prefill_tiles, once per call), and one CTA
// takes (tile, kv head): its two query heads x 64 rows are the M side of mma.sync m16n8k16 (one warp per
// 16 rows of a head), the slot's keys arrive 64 at a time in shared memory: S = Q K^T, online softmax in
// fp32 with the causal bound key <= row position, P rounded to bf16, O += P V (V through ldmatrix.trans).
// Keys before the call's first position come from the cache as earlier calls left them, the call's own
// keys were appended by the QKV epilogue before this kernel runs (flash_attn_with_kvcache semantics,
// src/vui/model.py:247-257; the prefill is driven by src/vui/engine.py:674-694).
//
// A row's result depends only on its own position and the slot's keys, in key tiles that always start at
// multiples of 64 from position 0: cutting a prompt into several calls does not change a bit.
#pragma once
#include "decode_kernels.cuh"

namespace vuib {

constexpr int PA_TILE = 64;       // query rows per tile, keys per step
constexpr int PA_KS = HD + 8;     // padded row stride of K / V tiles in shared memory (elements)

// tiles[2i] = first row of tile i, tiles[2i+1] = its rows (<= 64); tiles of one run of consecutive positions
// of one slot never straddle runs.  *n_tiles gets the count.  One CTA; rows staged through shared memory.
static __global__ void __launch_bounds__(256) k_prefill_tiles(const int32_t* __restrict__ row_slot,
                                                              const int32_t* __restrict__ row_pos, int M,
                                                              int32_t* __restrict__ tiles, int32_t* __restrict__ n_tiles) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int32_t pt_start[];  // 1 where a run starts
    for (int r = threadIdx.x; r < M; r += blockDim.x)
        pt_start[r] = r == 0 || row_slot[r] != row_slot[r - 1] || row_pos[r] != row_pos[r - 1] + 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0, run0 = 0;
        for (int r = 0; r < M; ++r) {
            if (pt_start[r]) run0 = r;
            if (((r - run0) % PA_TILE) == 0) {
                if (n > 0) tiles[2 * (n - 1) + 1] = r - tiles[2 * (n - 1)];
                tiles[2 * n] = r;
                ++n;
            }
        }
        if (n > 0) tiles[2 * (n - 1) + 1] = M - tiles[2 * (n - 1)];
        *n_tiles = n;
    }
}

struct PrefillAttnArgs {
    const bf16* q;        // (M, Hq*64), RoPE applied
    const bf16* kc;       // (slots, max_seq, Hkv, 64) of this layer, the call's keys already appended
    const bf16* vc;
    const int32_t* row_slot;  // checked copies
    const int32_t* row_pos;
    const int32_t* tiles;
    const int32_t* n_tiles;
    bf16* out;            // (M, Hq*64)
    int Hq, Hkv, max_seq;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int G>  // query heads per kv head (1 or 2)
__global__ void __launch_bounds__(G * 128) k_prefill_attn(PrefillAttnArgs a) {
    __shared__ __align__(16) bf16 Ks[PA_TILE][PA_KS];
    __shared__ __align__(16) bf16 Vs[PA_TILE][PA_KS];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.y;
    const int hq = kvh * G + (warp >> 2);   // this warp's query head
    const int rb = warp & 3;                // its 16 rows of the tile
    const int n_tiles = __ldcg(a.n_tiles);
    const size_t pos_stride = (size_t)a.Hkv * HD;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int row0 = __ldcg(a.tiles + 2 * tile), nrows = __ldcg(a.tiles + 2 * tile + 1);
        const int slot = __ldcg(a.row_slot + row0), pos0 = __ldcg(a.row_pos + row0);
        const int n_keys = pos0 + nrows;
        // rows of this thread: r_lo = rb*16 + g, r_hi = r_lo + 8 (inside the tile)
        const int r_lo = rb * 16 + g, r_hi = r_lo + 8;
        const bool ok_lo = r_lo < nrows, ok_hi = r_hi < nrows;
        // Q fragments: 4 k-steps of 16 dims
        uint32_t qa[4][4];
        {
            const bf16* q_lo = a.q + (size_t)(row0 + (ok_lo ? r_lo : 0)) * a.Hq * HD + hq * HD;
            const bf16* q_hi = a.q + (size_t)(row0 + (ok_hi ? r_hi : 0)) * a.Hq * HD + hq * HD;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                qa[ks][0] = ok_lo ? __ldcg(reinterpret_cast<const uint32_t*>(q_lo + ks * 16 + 2 * t)) : 0u;
                qa[ks][1] = ok_hi ? __ldcg(reinterpret_cast<const uint32_t*>(q_hi + ks * 16 + 2 * t)) : 0u;
                qa[ks][2] = ok_lo ? __ldcg(reinterpret_cast<const uint32_t*>(q_lo + ks * 16 + 8 + 2 * t)) : 0u;
                qa[ks][3] = ok_hi ? __ldcg(reinterpret_cast<const uint32_t*>(q_hi + ks * 16 + 8 + 2 * t)) : 0u;
            }
        }
        float m_lo = NEG_BIG, m_hi = NEG_BIG, l_lo = 0.f, l_hi = 0.f;
        float o[8][4];
#pragma unroll
        for (int dn = 0; dn < 8; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
        const bf16* kbase = a.kc + (size_t)slot * a.max_seq * pos_stride + kvh * HD;
        const bf16* vbase = a.vc + (size_t)slot * a.max_seq * pos_stride + kvh * HD;
        for (int k0 = 0; k0 < n_keys; k0 += PA_TILE) {
            __syncthreads();  // the previous key tile is used up
            for (int i = tid; i < PA_TILE * 8; i += G * 128) {
                const int key = i >> 3, ch = i & 7;
                const bool ok = k0 + key < n_keys;
                const size_t off = (size_t)(k0 + (ok ? key : 0)) * pos_stride + ch * 8;
                *reinterpret_cast<uint4*>(&Ks[key][ch * 8]) = ok ? ldg_stream(kbase + off) : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(&Vs[key][ch * 8]) = ok ? ldg_stream(vbase + off) : make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
            // whole tiles beyond this warp's last row position are masked: skip them (uniform per warp)
            const int warp_last = pos0 + min(rb * 16 + 15, nrows - 1);
            if (rb * 16 >= nrows || k0 > warp_last) continue;
            // ---- S = Q K^T for 64 keys: 8 n-tiles x 4 k-steps
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
                for (int kp = 0; kp < 2; ++kp) {  // two k-steps per ldmatrix.x4
                    uint32_t b0, b1, b2, b3;
                    // lanes 0-7: keys nt*8.., dims kp*32 + 0..7; 8-15: +8; 16-23: +16; 24-31: +24
                    const bf16* p = &Ks[nt * 8 + (lane & 7)][kp * 32 + (lane >> 3) * 8];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(s[nt][0]), "+f"(s[nt][1]), "+f"(s[nt][2]), "+f"(s[nt][3])
                                 : "r"(qa[2 * kp][0]), "r"(qa[2 * kp][1]), "r"(qa[2 * kp][2]), "r"(qa[2 * kp][3]), "r"(b0), "r"(b1));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(s[nt][0]), "+f"(s[nt][1]), "+f"(s[nt][2]), "+f"(s[nt][3])
                                 : "r"(qa[2 * kp + 1][0]), "r"(qa[2 * kp + 1][1]), "r"(qa[2 * kp + 1][2]), "r"(qa[2 * kp + 1][3]), "r"(b2), "r"(b3));
                }
            }
            // ---- scale, causal mask, online softmax (rows r_lo / r_hi of this thread, a quad shares a row)
            const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;
            float mx_lo = NEG_BIG, mx_hi = NEG_BIG;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = k0 + nt * 8 + 2 * t + (i & 1);
                    const bool hi = i >> 1;
                    const bool ok = key <= (hi ? p_hi : p_lo) && (hi ? ok_hi : ok_lo);
                    s[nt][i] = ok ? s[nt][i] * 0.125f : NEG_BIG;
                    if (hi) mx_hi = fmaxf(mx_hi, s[nt][i]);
                    else mx_lo = fmaxf(mx_lo, s[nt][i]);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float c_lo = __expf(m_lo - mn_lo), c_hi = __expf(m_hi - mn_hi);
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const bool hi = i >> 1;
                    // a masked score is NEG_BIG: exp underflows to exactly 0 against any real maximum
                    const float p = s[nt][i] <= 0.5f * NEG_BIG ? 0.f : __expf(s[nt][i] - (hi ? mn_hi : mn_lo));
                    s[nt][i] = p;
                    if (hi) sum_hi += p;
                    else sum_lo += p;
                }
            sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
            sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
            sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
            sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
            l_lo = l_lo * c_lo + sum_lo;
            l_hi = l_hi * c_hi + sum_hi;
            m_lo = mn_lo;
            m_hi = mn_hi;
#pragma unroll
            for (int dn = 0; dn < 8; ++dn) {
                o[dn][0] *= c_lo; o[dn][1] *= c_lo;
                o[dn][2] *= c_hi; o[dn][3] *= c_hi;
            }
            // ---- O += P V: P (bf16) as the A operand, 4 k-steps of 16 keys; V through ldmatrix.trans
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t pa0 = pack_bf16x2(s[2 * j][0], s[2 * j][1]), pa1 = pack_bf16x2(s[2 * j][2], s[2 * j][3]);
                const uint32_t pa2 = pack_bf16x2(s[2 * j + 1][0], s[2 * j + 1][1]), pa3 = pack_bf16x2(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
                for (int dp = 0; dp < 4; ++dp) {  // two 8-dim n-tiles per ldmatrix.x4.trans
                    uint32_t b0, b1, b2, b3;
                    // lanes 0-7: keys j*16 + 0..7, dims dp*16 + 0..7; 8-15: keys +8; 16-23: dims +8; 24-31: keys +8, dims +8
                    const bf16* p = &Vs[j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][dp * 16 + (lane >> 4) * 8];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(o[2 * dp][0]), "+f"(o[2 * dp][1]), "+f"(o[2 * dp][2]), "+f"(o[2 * dp][3])
                                 : "r"(pa0), "r"(pa1), "r"(pa2), "r"(pa3), "r"(b0), "r"(b1));
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                                 : "+f"(o[2 * dp + 1][0]), "+f"(o[2 * dp + 1][1]), "+f"(o[2 * dp + 1][2]), "+f"(o[2 * dp + 1][3])
                                 : "r"(pa0), "r"(pa1), "r"(pa2), "r"(pa3), "r"(b2), "r"(b3));
                }
            }
        }
        // ---- normalise and store
        if (ok_lo) {
            const float inv = 1.f / l_lo;
            bf16* dst = a.out + (size_t)(row0 + r_lo) * a.Hq * HD + hq * HD;
#pragma unroll
            for (int dn = 0; dn < 8; ++dn)
                *reinterpret_cast<uint32_t*>(dst + dn * 8 + 2 * t) = pack_bf16x2(o[dn][0] * inv, o[dn][1] * inv);
        }
        if (ok_hi) {
            const float inv = 1.f / l_hi;
            bf16* dst = a.out + (size_t)(row0 + r_hi) * a.Hq * HD + hq * HD;
#pragma unroll
            for (int dn = 0; dn < 8; ++dn)
                *reinterpret_cast<uint32_t*>(dst + dn * 8 + 2 * t) = pack_bf16x2(o[dn][2] * inv, o[dn][3] * inv);
        }
    }
}

}  // namespace vuib
