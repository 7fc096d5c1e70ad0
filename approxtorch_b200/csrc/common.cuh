// Shared helpers of the C-ABI library: status codes, per-thread error text, launch checks,
// operand-to-index conversion and the LUT image layout.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/approxtorch_b200.h"

namespace atb {

void set_error(const char* fmt, ...);

inline int fail_invalid(const char* what)
{
    set_error("invalid argument: %s", what);
    return ATB_ERR_INVALID;
}

inline int check_launch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return ATB_ERR_CUDA;
    }
    return ATB_OK;
}

#define ATB_REQUIRE(cond, what) \
    do { if (!(cond)) return ::atb::fail_invalid(what); } while (0)

inline bool aligned_to(const void* p, uintptr_t bytes)
{
    return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0;
}

inline int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

int sm_count();

// ---------------------------------------------------------------------------------------------
// LUT image: what atb_lut_prepare writes and every LUT kernel reads.
//   flags[0] != 0 : table is NOT exactly representable as int16 (integer, |v| <= 32767)
//   flags[1] != 0 : table is NOT exactly representable as uint16 (integer, 0 <= v <= 65535)
// The 16-bit images hold the low 16 bits of the integer value, valid under either reading.
// "T" images are transposed: entry [w][x].
// ---------------------------------------------------------------------------------------------
struct LutImage {
    int flags[4];
    // tabTP16: transposed and x-permuted; for the int16 class stored with bit 15 of every entry flipped
    // (value + 32768 as an unsigned entry).  A 32-bit word of row w holds the pair i = {x = i (low half),
    // x = i + 128 (high half)}, i = 0..127, and pair i is word 4 * (i & 31) + (i >> 5) of the row, so that lane l
    // of a warp reads the pairs l, l + 32, l + 64, l + 96 with one 16-byte load
    int16_t tabTP16[65536];
    int16_t tabT16[65536];
    int16_t tab16[65536];
    float tabT32[65536];
    float tab32[65536];
    // tabTP32: transposed ([w][x]) and x-permuted within each half-row of 128 for the fp32 staging loads: position
    // h*128 + 4*l + e of row w holds x = h*128 + l + 32*e, so that lane l of a staging warp gets the four entries
    // x = l, l+32, l+64, l+96 of its half-row with one 16-byte load
    float tabTP32[65536];
};

enum LutClass { LUT_I16 = 0, LUT_U16 = 1, LUT_F32 = 2 };

__device__ __forceinline__ int lut_class_of(const LutImage* img)
{
    if (__ldg(&img->flags[0]) == 0) return LUT_I16;
    if (__ldg(&img->flags[1]) == 0) return LUT_U16;
    return LUT_F32;
}

// fp32 integer-valued operand -> LUT index: round half to even, add offset, saturate to [0,255]
__device__ __forceinline__ uint8_t index_from_float(float v, int offset)
{
    int q = __float2int_rn(v) + offset;
    q = max(0, min(255, q));
    return static_cast<uint8_t>(q);
}

// index of an already-quantised element by storage type: fp32 value / int8 value / uint8 index
template <int DT>
__device__ __forceinline__ int index_of(const void* base, long long i)
{
    if constexpr (DT == ATB_F32) {
        int q = __float2int_rn(static_cast<const float*>(base)[i]);
        return max(-128, min(127, q)) + 128;
    } else if constexpr (DT == ATB_I8) {
        return static_cast<int>(static_cast<const int8_t*>(base)[i]) + 128;
    } else {
        return static_cast<int>(static_cast<const uint8_t*>(base)[i]);
    }
}

// implicit-im2col geometry shared by the conv kernels
struct ConvGeom {
    int C, H, W, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW;
};

inline bool conv_out_shape(int H, int W, int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw,
                           int* OH, int* OW)
{
    if (kh < 1 || kw < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0 || dh < 1 || dw < 1) return false;
    const long long oh = (static_cast<long long>(H) + 2LL * ph - static_cast<long long>(dh) * (kh - 1) - 1) / sh + 1;
    const long long ow = (static_cast<long long>(W) + 2LL * pw - static_cast<long long>(dw) * (kw - 1) - 1) / sw + 1;
    if (static_cast<long long>(H) + 2LL * ph - static_cast<long long>(dh) * (kh - 1) - 1 < 0) return false;
    if (static_cast<long long>(W) + 2LL * pw - static_cast<long long>(dw) * (kw - 1) - 1 < 0) return false;
    if (oh < 1 || ow < 1) return false;
    *OH = static_cast<int>(oh);
    *OW = static_cast<int>(ow);
    return true;
}

// Forward LUT GEMM on a table of the fp32 class, run by the cluster kernel of pair_grad.cu (filled in by lut_gemm.cu)
struct PairFwdParams {
    const uint8_t* x;
    const uint8_t* w;
    const float* tab;          // LutImage::tabTP32
    float* y;
    long long R;
    int K, L, O;
    int image_mode, x_xor, pad_index;
    ConvGeom g;
    const float* alpha;
    const float* beta;
    const float* zero_x;
    const float* zero_w;
    const int* wsum;
};
int pair_forward_launch(const PairFwdParams& p, int mode, cudaStream_t stream);

// STE / LRE image-space backward on the tensor cores (tc_grad.cu); used by atb_lre_conv_bwd
int tc_conv_grad_w(const float* go, const void* x, int x_dtype, const float* dw, const float* go_scale, float* grad_w,
                   int N, int O, const ConvGeom& g, int pad_index, bool exact_tables, cudaStream_t s);
int tc_conv_grad_x(const float* go, const uint8_t* widx, const float* dx, const float* go_scale, const float* w_zero,
                   const uint8_t* x_mask, const float* x_scale, float* grad_x, int N, int O, const ConvGeom& g,
                   bool exact_tables, cudaStream_t s);
int tc_status_read(int* status);
size_t tc_packed_scratch_bytes(int N, int O, const ConvGeom& g, bool need_x, bool need_w, bool exact_tables, bool deterministic);
int tc_packed_conv_bwd(const float* go, const void* x, int x_dtype, const uint8_t* widx, const float* dx, const float* dw,
                       const float* go_scale, const float* w_zero, const uint8_t* x_mask, const float* x_scale,
                       float* grad_x, float* grad_w, int N, int O, const ConvGeom& g, int pad_index, bool exact_tables,
                       bool deterministic, void* scratch, cudaStream_t s);

inline int grid_for(long long work, int threads, int cap)
{
    long long b = (work + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > cap) b = cap;
    return static_cast<int>(b);
}

}  // namespace atb
