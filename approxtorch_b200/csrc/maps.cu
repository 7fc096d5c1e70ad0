// Index unfold (im2col to uint8 LUT indices) and 256-entry table maps.  Streaming kernels:
// one pass over the output, table in shared memory, 4-wide stores where alignment allows.
#include "common.cuh"

namespace atb {

constexpr int kThreads = 256;

// out[n, k, l]: k = (c, i, j), l = (oh, ow).  One thread produces 4 consecutive l of one (n, k) row
// when L % 4 == 0 (a single uchar4 store), else one element.
template <int DT, int VEC>
__global__ void im2col_u8_kernel(const void* __restrict__ x, uint8_t* __restrict__ out, int N, ConvGeom g, int pad_index)
{
    const int L = g.OH * g.OW;
    const int K = g.C * g.KH * g.KW;
    const int LV = L / VEC;
    const long long total = static_cast<long long>(N) * K * LV;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int lv = static_cast<int>(t % LV);
        const long long nk = t / LV;
        const int k = static_cast<int>(nk % K);
        const long long n = nk / K;
        const int c = k / (g.KH * g.KW);
        const int rem = k - c * (g.KH * g.KW);
        const int i = rem / g.KW;
        const int j = rem - i * g.KW;
        const long long plane = (n * g.C + c) * g.H;
        int l = lv * VEC;
        int oh = l / g.OW;
        int ow = l - oh * g.OW;
        uint8_t vals[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const int ih = oh * g.SH - g.PH + i * g.DH;
            const int iw = ow * g.SW - g.PW + j * g.DW;
            int idx = pad_index;
            if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
                idx = index_of<DT>(x, (plane + ih) * g.W + iw);
            vals[e] = static_cast<uint8_t>(idx);
            if (++ow == g.OW) { ow = 0; ++oh; }
        }
        uint8_t* dst = out + (n * K + k) * static_cast<long long>(L) + l;
        if constexpr (VEC == 4) *reinterpret_cast<uchar4*>(dst) = make_uchar4(vals[0], vals[1], vals[2], vals[3]);
        else dst[0] = vals[0];
    }
}

template <int DT>
__global__ void lut_map_kernel(const void* __restrict__ x, const float* __restrict__ table, float* __restrict__ out,
                               long long numel, bool vec)
{
    __shared__ float st[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) st[i] = table[i];
    __syncthreads();
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = vec ? (numel >> 2) : 0;
    for (long long i = t0; i < n4; i += stride) {
        float4 r;
        r.x = st[index_of<DT>(x, 4 * i)]; r.y = st[index_of<DT>(x, 4 * i + 1)];
        r.z = st[index_of<DT>(x, 4 * i + 2)]; r.w = st[index_of<DT>(x, 4 * i + 3)];
        reinterpret_cast<float4*>(out)[i] = r;
    }
    for (long long i = (n4 << 2) + t0; i < numel; i += stride) out[i] = st[index_of<DT>(x, i)];
}

template <int DT>
__global__ void lut_map_pad_kernel(const void* __restrict__ x, const float* __restrict__ table, float* __restrict__ out,
                                   long long planes, int H, int W, int PH, int PW)
{
    __shared__ float st[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) st[i] = table[i];
    __syncthreads();
    const int WP = W + 2 * PW;
    const long long hw = static_cast<long long>(H + 2 * PH) * WP;
    const long long total = planes * hw;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
        const long long p = t / hw;
        const int q = static_cast<int>(t - p * hw);
        const int h = q / WP - PH;
        const int w = q % WP - PW;
        float v = st[128];
        if (static_cast<unsigned>(h) < static_cast<unsigned>(H) && static_cast<unsigned>(w) < static_cast<unsigned>(W))
            v = st[index_of<DT>(x, (p * H + h) * W + w)];
        out[t] = v;
    }
}

}  // namespace atb

using namespace atb;

#define ATB_DISPATCH_DTYPE(dtype, CALL)                     \
    switch (dtype) {                                        \
        case ATB_F32: { constexpr int DT = ATB_F32; CALL; break; } \
        case ATB_I8:  { constexpr int DT = ATB_I8;  CALL; break; } \
        case ATB_U8:  { constexpr int DT = ATB_U8;  CALL; break; } \
        default: return fail_invalid("dtype must be ATB_F32, ATB_I8 or ATB_U8"); \
    }

extern "C" int atb_im2col_u8(const void* x, int dtype, int N, int C, int H, int W, int kh, int kw, int sh, int sw,
                             int ph, int pw, int dh, int dw, int pad_index, uint8_t* out, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0, "negative dimension");
    ATB_REQUIRE(pad_index >= 0 && pad_index <= 255, "pad_index out of range");
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw, &OH, &OW), "conv geometry yields empty output");
    const long long total = static_cast<long long>(N) * C * kh * kw * OH * OW;
    if (total == 0) return ATB_OK;
    ATB_REQUIRE(x && out, "null pointer");
    ATB_REQUIRE(static_cast<long long>(OH) * OW <= 2147483647LL && static_cast<long long>(C) * kh * kw <= 2147483647LL,
                "dimensions too large");
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = ((OH * OW) % 4 == 0) && aligned_to(out, 4);
    const int grid = grid_for(vec ? total / 4 : total, kThreads, 32 * sm_count());
    if (vec) { ATB_DISPATCH_DTYPE(dtype, (im2col_u8_kernel<DT, 4><<<grid, kThreads, 0, s>>>(x, out, N, g, pad_index))) }
    else { ATB_DISPATCH_DTYPE(dtype, (im2col_u8_kernel<DT, 1><<<grid, kThreads, 0, s>>>(x, out, N, g, pad_index))) }
    return check_launch("im2col_u8_kernel");
}

extern "C" int atb_lut_map(const void* x, int dtype, const float* table, float* out, long long numel, void* stream)
{
    ATB_REQUIRE(numel >= 0, "negative numel");
    if (numel == 0) return ATB_OK;
    ATB_REQUIRE(x && table && out, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = aligned_to(out, 16);
    const int grid = grid_for(vec ? numel / 4 + 1 : numel, kThreads, 16 * sm_count());
    ATB_DISPATCH_DTYPE(dtype, (lut_map_kernel<DT><<<grid, kThreads, 0, s>>>(x, table, out, numel, vec)))
    return check_launch("lut_map_kernel");
}

extern "C" int atb_lut_map_pad(const void* x, int dtype, const float* table, float* out, int N, int C, int H, int W,
                               int ph, int pw, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0 && ph >= 0 && pw >= 0, "negative dimension");
    const long long total = static_cast<long long>(N) * C * (H + 2LL * ph) * (W + 2LL * pw);
    if (total == 0) return ATB_OK;
    ATB_REQUIRE(table && out && (static_cast<long long>(N) * C * H * W == 0 || x), "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_for(total, kThreads, 16 * sm_count());
    ATB_DISPATCH_DTYPE(dtype, (lut_map_pad_kernel<DT><<<grid, kThreads, 0, s>>>(x, table, out, static_cast<long long>(N) * C, H, W, ph, pw)))
    return check_launch("lut_map_pad_kernel");
}
