// Warp-level 32 x 32 bit-matrix transpose, shared by the bit-frame kernels.
#pragma once

#include <cstdint>

namespace bb200 {

// 32 x 32 bit-matrix transpose across a warp: lane k holds row k; afterwards lane j holds column j (bit k of the result =
// bit j of lane k's word).  Five exchange stages: at distance s the lanes r and r + s swap the off-diagonal s x s blocks of every
// 2s x 2s block (bits with (c & s) != 0 of the lower lane against bits with (c & s) == 0 of the upper one).  The partner's word is
// rotated by s (lower lane) or 32 - s (upper lane) -- inside the bits that are taken a rotation equals the shift -- and merged by
// one bit-select: a shuffle, a funnel shift and a logic operation per stage instead of 32 ballots.
struct BitTranspose {
    uint32_t keep[5];          // bits a lane keeps at stage k
    int rot[5];                // left rotation of the partner's word at stage k
    __device__ __forceinline__ explicit BitTranspose(int lane)
    {
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            const int s = 16 >> k;
            const uint32_t low = k == 0 ? 0x0000ffffu : k == 1 ? 0x00ff00ffu : k == 2 ? 0x0f0f0f0fu : k == 3 ? 0x33333333u : 0x55555555u;
            keep[k] = (lane & s) ? ~low : low;
            rot[k]  = (lane & s) ? 32 - s : s;
        }
    }
    __device__ __forceinline__ uint32_t operator()(uint32_t v) const
    {
#pragma unroll
        for (int k = 0; k < 5; ++k) {
            const uint32_t other = __shfl_xor_sync(0xffffffffu, v, 16 >> k);
            const uint32_t r = __funnelshift_l(other, other, rot[k]);
            v = (v & keep[k]) | (r & ~keep[k]);
        }
        return v;
    }
};

}   // namespace bb200
