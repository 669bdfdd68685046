// The register-level core of the BitLinear decode kernels: packed ternary words straight into
// mma.sync.m16n8k32.u8.s8 operands.
#pragma once
#include "common.cuh"

namespace nslq {

static __device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Accumulators of one token tile: class i collects the trits in position i of their byte,
// whose codes are used as they sit in the byte, i.e. scaled by 64, 16, 4, 1.
struct Acc4 { int v[4][4]; };

static __device__ __forceinline__ void acc_zero(Acc4 &a)
{
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) a.v[i][r] = 0;
}
// sum_k q*code for fragment register r: every class is an exact multiple of its scale.
static __device__ __forceinline__ int acc_value(const Acc4 &a, int r)
{
    return (a.v[0][r] >> 6) + (a.v[1][r] >> 4) + (a.v[2][r] >> 2) + a.v[3][r];
}

// One 64-trit chunk of rows g and g+8 (ra, rb) against the matching 64 int8 activations of
// one token tile (xq[0..3], consumption order): 8 MMAs.  A packed word w holds trit i of byte
// j in bits 8j+6-2i; `w & (0x03030303 << (6-2i))` is therefore the four codes of position i,
// each multiplied by 4^(3-i), still a valid u8 -- one AND per operand register and no shift.
// An MMA pairs the same position class of two words so that its sum has a single scale.
static __device__ __forceinline__ void chunk_mma(Acc4 &acc, const uint4 &ra, const uint4 &rb, const uint4 (&xq)[4])
{
    const uint32_t wwa[4] = {ra.x, ra.y, ra.z, ra.w};
    const uint32_t wwb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
    for (int jp = 0; jp < 4; jp += 2) {
        const uint32_t x0[4] = {xq[jp].x, xq[jp].y, xq[jp].z, xq[jp].w};
        const uint32_t x1[4] = {xq[jp + 1].x, xq[jp + 1].y, xq[jp + 1].z, xq[jp + 1].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t mask = 0x03030303u << (6 - 2 * i);
            mma_u8s8(acc.v[i], wwa[jp] & mask, wwb[jp] & mask, wwa[jp + 1] & mask, wwb[jp + 1] & mask, x0[i], x1[i]);
        }
    }
}

// The same chunk with the two word pairs on separate accumulators: eight independent MMA chains
// instead of four.  A dependent mma.sync issues only some hundreds of cycles after its producer
// on this part, so a warp needs that many chains in flight to keep the pipe busy.
static __device__ __forceinline__ void chunk_mma2(Acc4 &acc0, Acc4 &acc1, const uint4 &ra, const uint4 &rb, const uint4 (&xq)[4])
{
    const uint32_t wwa[4] = {ra.x, ra.y, ra.z, ra.w};
    const uint32_t wwb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
    for (int jp = 0; jp < 4; jp += 2) {
        const uint32_t x0[4] = {xq[jp].x, xq[jp].y, xq[jp].z, xq[jp].w};
        const uint32_t x1[4] = {xq[jp + 1].x, xq[jp + 1].y, xq[jp + 1].z, xq[jp + 1].w};
        Acc4 &acc = jp ? acc1 : acc0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t mask = 0x03030303u << (6 - 2 * i);
            mma_u8s8(acc.v[i], wwa[jp] & mask, wwb[jp] & mask, wwa[jp + 1] & mask, wwb[jp + 1] & mask, x0[i], x1[i]);
        }
    }
}

}  // namespace nslq
