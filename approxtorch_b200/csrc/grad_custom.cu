// Custom-pair gradient backward (one surrogate derivative per (x, w) pair, two 256x256 fp32 tables)
// and the depthwise LUT convolution forward.
//
//   grad_x[n,k,l] = sum_o dY[n,o,l] * DX[x[n,k,l]][w[o,k]]
//   grad_w[o,k]   = sum_{n,l} dY[n,o,l] * DW[x[n,k,l]][w[o,k]]
//
// Both are 2-D gathers from a 256 KB fp32 table (too large for one SM's shared memory together with
// operand tiles), so the table stays in global memory behind the read-only L1/L2 path and the kernels
// are organised to make every fetched operand byte and dY value serve many lookups.
#include "common.cuh"

namespace atb {

// ---- grad_x: block = 64 pixels x 8 reduction rows; output channels swept in tiles of 32 ----------
constexpr int DXL = 64, DXK = 8, DXO = 32;

__global__ void __launch_bounds__(DXL * DXK) custom_dx_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w,
                                                              const float* __restrict__ dy, const float* __restrict__ tab,
                                                              float* __restrict__ gx, int K, int L, int O)
{
    __shared__ float s_dy[DXO][DXL];
    __shared__ uint8_t s_w[DXO][DXK];
    const int tl = threadIdx.x, tk = threadIdx.y;
    const int l = blockIdx.x * DXL + tl;
    const int k = blockIdx.y * DXK + tk;
    const long long n = blockIdx.z;
    const bool live = (l < L) && (k < K);
    const float* row = tab + (live ? (static_cast<int>(x[(n * K + k) * L + l]) << 8) : 0);
    const int tid = tk * DXL + tl;
    float acc = 0.0f;
    for (int o0 = 0; o0 < O; o0 += DXO) {
        for (int e = tid; e < DXO * DXL; e += DXL * DXK) {
            const int oo = e / DXL, ll = e % DXL;
            const int og = o0 + oo, lg = blockIdx.x * DXL + ll;
            s_dy[oo][ll] = (og < O && lg < L) ? dy[(n * O + og) * L + lg] : 0.0f;
        }
        for (int e = tid; e < DXO * DXK; e += DXL * DXK) {
            const int oo = e / DXK, kk = e % DXK;
            const int og = o0 + oo, kg = blockIdx.y * DXK + kk;
            s_w[oo][kk] = (og < O && kg < K) ? w[static_cast<long long>(og) * K + kg] : 0;
        }
        __syncthreads();
        if (live) {
            const int lim = min(DXO, O - o0);
            for (int oo = 0; oo < lim; ++oo) acc = fmaf(s_dy[oo][tl], __ldg(row + s_w[oo][tk]), acc);
        }
        __syncthreads();
    }
    if (live) gx[(n * K + k) * L + l] = acc;
}

// ---- grad_w: block = one reduction row k x 8 output channels; 256 threads sweep all pixels -------
constexpr int DWO = 8, DWT = 256;

__global__ void __launch_bounds__(DWT) custom_dw_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w,
                                                        const float* __restrict__ dy, const float* __restrict__ tab,
                                                        float* __restrict__ gw, int N, int K, int L, int O)
{
    __shared__ float s_col[DWO][257];
    __shared__ float s_red[DWO][DWT / 32];
    const int k = blockIdx.x;
    const int o0 = blockIdx.y * DWO;
    const int tid = threadIdx.x;
    for (int e = tid; e < DWO * 256; e += DWT) {
        const int oo = e >> 8, a = e & 255;
        const int og = min(o0 + oo, O - 1);
        s_col[oo][a] = tab[(a << 8) + w[static_cast<long long>(og) * K + k]];
    }
    __syncthreads();
    float acc[DWO];
#pragma unroll
    for (int oo = 0; oo < DWO; ++oo) acc[oo] = 0.0f;
    const long long P = static_cast<long long>(N) * L;
    for (long long p = tid; p < P; p += DWT) {
        const long long n = p / L;
        const long long l = p - n * L;
        const int a = x[(n * K + k) * L + l];
        const float* dyn = dy + (n * O + o0) * L + l;
#pragma unroll
        for (int oo = 0; oo < DWO; ++oo)
            if (o0 + oo < O) acc[oo] = fmaf(dyn[static_cast<long long>(oo) * L], s_col[oo][a], acc[oo]);
    }
#pragma unroll
    for (int oo = 0; oo < DWO; ++oo) {
        float v = acc[oo];
        for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
        if ((tid & 31) == 0) s_red[oo][tid >> 5] = v;
    }
    __syncthreads();
    if (tid < DWO && o0 + tid < O) {
        float v = 0.0f;
        for (int i = 0; i < DWT / 32; ++i) v += s_red[tid][i];
        gw[static_cast<long long>(o0 + tid) * K + k] = v;
    }
}

// ---- depthwise LUT conv forward: one thread per output, taps in ascending (i, j) order -------------
template <int DT>
__global__ void dwconv_kernel(const void* __restrict__ x, const uint8_t* __restrict__ widx, const LutImage* __restrict__ img,
                              float* __restrict__ y, int N, ConvGeom g, int pad_index)
{
    const int cls = lut_class_of(img);
    const long long total = static_cast<long long>(N) * g.C * g.OH * g.OW;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const int taps = g.KH * g.KW;
    for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int ow = static_cast<int>(t % g.OW);
        const long long t1 = t / g.OW;
        const int oh = static_cast<int>(t1 % g.OH);
        const long long nc = t1 / g.OH;
        const int c = static_cast<int>(nc % g.C);
        const uint8_t* wc = widx + static_cast<long long>(c) * taps;
        long long isum = 0;
        float fsum = 0.0f;
        for (int i = 0; i < g.KH; ++i) {
            const int ih = oh * g.SH - g.PH + i * g.DH;
            for (int j = 0; j < g.KW; ++j) {
                const int iw = ow * g.SW - g.PW + j * g.DW;
                int xi = pad_index;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
                    xi = index_of<DT>(x, (nc * g.H + ih) * g.W + iw);
                const int flat = (xi << 8) | wc[i * g.KW + j];
                if (cls == LUT_I16) isum += __ldg(img->tab16 + flat);
                else if (cls == LUT_U16) isum += static_cast<uint16_t>(__ldg(img->tab16 + flat));
                else fsum += __ldg(img->tab32 + flat);
            }
        }
        y[t] = (cls == LUT_F32) ? fsum : static_cast<float>(isum);
    }
}

}  // namespace atb

using namespace atb;

extern "C" int atb_custom_bwd_dx(const uint8_t* x, const uint8_t* w, const float* dy, const float* dx_lut,
                                 float* grad_x, int N, int K, int L, int O, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    if (static_cast<long long>(N) * K * L == 0) return ATB_OK;
    ATB_REQUIRE(x && grad_x && dx_lut && (O == 0 || (w && dy)), "null pointer");
    ATB_REQUIRE(N <= 65535 && ceil_div(K, DXK) <= 65535, "N or K too large");
    dim3 block(DXL, DXK), grid(ceil_div(L, DXL), ceil_div(K, DXK), N);
    custom_dx_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(x, w, dy, dx_lut, grad_x, K, L, O);
    return check_launch("custom_dx_kernel");
}

extern "C" int atb_custom_bwd_dw(const uint8_t* x, const uint8_t* w, const float* dy, const float* dw_lut,
                                 float* grad_w, int N, int K, int L, int O, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    if (static_cast<long long>(O) * K == 0) return ATB_OK;
    ATB_REQUIRE(w && grad_w && dw_lut && (static_cast<long long>(N) * L == 0 || (x && dy)), "null pointer");
    ATB_REQUIRE(ceil_div(O, DWO) <= 65535, "O too large");
    dim3 grid(K, ceil_div(O, DWO));
    custom_dw_kernel<<<grid, DWT, 0, static_cast<cudaStream_t>(stream)>>>(x, w, dy, dw_lut, grad_w, N, K, L, O);
    return check_launch("custom_dw_kernel");
}

extern "C" int atb_lut_dwconv_fwd(const void* x, int dtype, const uint8_t* widx, const void* lut_image, float* y,
                                  int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
                                  int dh, int dw, int pad_index, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0, "negative dimension");
    ATB_REQUIRE(pad_index >= 0 && pad_index <= 255, "pad_index out of range");
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw, &OH, &OW), "conv geometry yields empty output");
    const long long total = static_cast<long long>(N) * C * OH * OW;
    if (total == 0) return ATB_OK;
    ATB_REQUIRE(x && widx && lut_image && y, "null pointer");
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_for(total, 256, 32 * sm_count());
    const LutImage* img = static_cast<const LutImage*>(lut_image);
    switch (dtype) {
        case ATB_F32: dwconv_kernel<ATB_F32><<<grid, 256, 0, s>>>(x, widx, img, y, N, g, pad_index); break;
        case ATB_I8: dwconv_kernel<ATB_I8><<<grid, 256, 0, s>>>(x, widx, img, y, N, g, pad_index); break;
        case ATB_U8: dwconv_kernel<ATB_U8><<<grid, 256, 0, s>>>(x, widx, img, y, N, g, pad_index); break;
        default: return fail_invalid("dtype must be ATB_F32, ATB_I8 or ATB_U8");
    }
    return check_launch("dwconv_kernel");
}
