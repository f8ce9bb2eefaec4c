// Interface between the engine (vuib200.cu) and the barrier-free persistent frame kernel
// (frame_ll.cu), which is a translation unit of its own.
#pragma once
#include <cuda_runtime.h>

#include "frame_kernel.cuh"

namespace vuib {

constexpr int LL_MAXB = 4;  // streams per launch

// Word offsets of the tagged exchange buffers (32-bit words: bf16 payload | 16-bit tag << 16).
// The sizes are those of the one model shape the kernel is built for: d 1024, ffn 3072,
// 16/8 heads of 64, codebooks of 2048, depth transformer 512 wide, <= 1536 ffn, 4 layers, 16 positions.
struct LLLayout {
    static constexpr size_t D = 1024, F = 3072, CS = 2048, RD = 512, RQF = 1536, Q = 16, RL = 4;
    static constexpr size_t CB0_STRIDE = CS + 8;  // word CS of a row is the EOS logit
    static constexpr size_t X = 0;
    static constexpr size_t QO = X + LL_MAXB * D;
    static constexpr size_t KV = QO + LL_MAXB * D;  // new k (512) | new v (512) per row
    static constexpr size_t ATT = KV + LL_MAXB * D;
    static constexpr size_t ACT = ATT + LL_MAXB * D;
    static constexpr size_t HID = ACT + LL_MAXB * F;
    static constexpr size_t CB0 = HID + LL_MAXB * D;
    static constexpr size_t RX2 = CB0 + LL_MAXB * CB0_STRIDE;
    static constexpr size_t RX = RX2 + 2 * LL_MAXB * RD;
    static constexpr size_t RQ = RX + LL_MAXB * RD;
    static constexpr size_t RACT = RQ + 2 * LL_MAXB * RD;
    static constexpr size_t RLOG = RACT + 2 * LL_MAXB * RQF;
    static constexpr size_t RK = RLOG + LL_MAXB * CS;
    static constexpr size_t RV = RK + RL * LL_MAXB * Q * RD;
    static constexpr size_t END = RV + RL * LL_MAXB * Q * RD;
};

struct LLArgs {
    FrameArgs fa;
    uint32_t* bufs;   // LLLayout::END words, zero at first use
    uint32_t* state;  // [0] phase counter, [1] (B, codebooks) of the last launch, [2] barrier counter; zero at first use
};

// Launches one frame (backbone + heads + depth step) for B <= LL_MAXB streams.  Returns a cudaError_t.
int launch_frame_ll(const LLArgs& a, int rq_ffn, int num_sms, bool cooperative, cudaStream_t s);

}  // namespace vuib
