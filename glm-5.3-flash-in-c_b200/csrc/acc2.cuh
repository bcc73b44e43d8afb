// acc2.cuh - running sums in two floats (sum, carry) instead of one double.
//
// The reference accumulates its dot products in FP64 (src/core/glm53f_ops.c:101-154 and every
// caller). On this GPU the FP64 pipe issues about 16 FMA per clock per SM (an eighth of the FP32
// rate; the MLA score kernel sustains 14.5), and a float -> double conversion costs about twice
// an FP64 FMA, so a loop that converts both factors of every product spends four fifths of its
// time converting. A compensated FP32 sum (Knuth's TwoSum for the addition, the FMA's exact
// product error for the product) costs ten FP32 instructions per term - less than half of
// convert + convert + FMA - and carries the sum to about 2^-46 relative: after the final rounding
// to float it equals the FP64 result except where that result sits within 2^-22 ulp of a
// rounding boundary. Used where the factors arrive as floats or BF16 (mHC mixer rows and
// stream expansion); kernels whose factors already sit in shared memory as doubles keep the FP64 FMA.
#pragma once

namespace g5b {

struct Acc2 {
    float s = 0.f, c = 0.f;
};

// a += p  (p a float)
__device__ __forceinline__ void acc2_add(Acc2 &a, float p)
{
    const float s = __fadd_rn(a.s, p);
    const float bb = __fsub_rn(s, a.s);
    const float e = __fadd_rn(__fsub_rn(a.s, __fsub_rn(s, bb)), __fsub_rn(p, bb));
    a.s = s;
    a.c = __fadd_rn(a.c, e);
}

// a += x * y, the product's own rounding error included
__device__ __forceinline__ void acc2_fma(Acc2 &a, float x, float y)
{
    const float p = __fmul_rn(x, y);
    const float pe = __fmaf_rn(x, y, -p);
    acc2_add(a, p);
    a.c = __fadd_rn(a.c, pe);
}

// a += (xh + xl) * y for a factor held as two floats (a double rounded to 48 bits)
__device__ __forceinline__ void acc2_fma2(Acc2 &a, float xh, float xl, float y)
{
    acc2_fma(a, xh, y);
    a.c = __fmaf_rn(xl, y, a.c);
}

__device__ __forceinline__ double acc2_f64(const Acc2 &a) { return (double)a.s + (double)a.c; }
__device__ __forceinline__ float acc2_f32(const Acc2 &a) { return __fadd_rn(a.s, a.c); }

}  // namespace g5b
