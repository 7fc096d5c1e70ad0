// Depthwise LUT convolution (groups == C, channel multiplier 1): forward and STE / LRE backward.
//
//   y[n,c,oh,ow]    = sum_{i,j} lut[x(n,c,ih,iw)][w(c,i,j)]                    taps outside the image look up pad_index
//   grad_x[n,c,h,w] = sum_{(i,j) reaching (h,w)} go[n,c,oh,ow] * dx[w(c,i,j)]
//   grad_w[c,(i,j)] = sum_{n,oh,ow} go[n,c,oh,ow] * dw[x(n,c,ih,iw) or pad_index]
//
// A channel only ever touches kh*kw columns of the table, so a block works on ONE channel: it copies those
// columns (kh*kw x 256 entries, 9 KB for 3x3) into shared memory once and then streams over the channel's output
// pixels of every sample, one output per thread, taps in ascending (i, j) order - the order a per-channel LUT GEMM
// would use, so the result is bit-identical to it (approxtorch/backend/csrc/claude/dwconv_claude.cu:78-266 keeps the
// same contract).  The kernels are bound by the 5 bytes per output they move (1 read, 4 written), not by the
// lookups.  The backward needs no table lookups beyond the two 256-entry slope tables: grad_x is a gather over the
// taps that reach a pixel, grad_w a per-channel reduction over all output pixels (one block per channel and slice
// of the pixels, block-wide tree sums, fp32 atomics across slices).
#include "common.cuh"

namespace atb {

constexpr int kDwThreads = 256;
constexpr int kDwMaxTaps = 49;            // up to 7x7 windows in shared memory; larger windows take the direct path

// ---- forward ----------------------------------------------------------------------------------------------------
// grid (C, slices): block (c, s) handles outputs p = s*chunk .. of channel c, p = (n, oh, ow) flattened.
template <int DT, bool SMEM>
__global__ void __launch_bounds__(kDwThreads) dwconv_fwd_kernel(const void* __restrict__ x, const uint8_t* __restrict__ widx,
                                                                const LutImage* __restrict__ img, float* __restrict__ y,
                                                                int N, ConvGeom g, int pad_index, long long chunk)
{
    extern __shared__ __align__(16) uint8_t dw_smem[];
    int* s_col = reinterpret_cast<int*>(dw_smem);                    // [taps][256] entry bits (int or float)
    const int cls = lut_class_of(img);
    const int c = blockIdx.x;
    const int taps = g.KH * g.KW;
    const uint8_t* wc = widx + static_cast<long long>(c) * taps;
    if (SMEM) {
        for (int e = threadIdx.x; e < taps * 256; e += blockDim.x) {
            const int t = e >> 8, xi = e & 255;
            const int flat = (static_cast<int>(wc[t]) << 8) | xi;      // transposed images: [w][x], coalesced over x
            int bits;
            if (cls == LUT_I16) bits = static_cast<int>(__ldg(img->tabT16 + flat));
            else if (cls == LUT_U16) bits = static_cast<int>(static_cast<uint16_t>(__ldg(img->tabT16 + flat)));
            else bits = __float_as_int(__ldg(img->tabT32 + flat));
            s_col[e] = bits;
        }
        __syncthreads();
    }
    // The slice [p_beg, p_end) of the channel's outputs p = n * L + l is walked sample by sample, so that the inner
    // loop needs no 64-bit division.
    const int L = g.OH * g.OW;
    const long long P = static_cast<long long>(N) * L;
    const long long p_beg = static_cast<long long>(blockIdx.y) * chunk;
    const long long p_end = min(P, p_beg + chunk);
    for (long long n = p_beg / L; n * L < p_end; ++n) {
        const int l_beg = static_cast<int>(max(p_beg - n * L, 0LL));
        const int l_end = static_cast<int>(min(p_end - n * L, static_cast<long long>(L)));
        const long long plane = (n * g.C + c) * g.H;
        float* yn = y + (n * g.C + c) * static_cast<long long>(L);
        for (int l = l_beg + threadIdx.x; l < l_end; l += blockDim.x) {
            const int oh = l / g.OW, ow = l - oh * g.OW;
            int isum = 0;                      // |sum| <= taps * 65535: fits
            float fsum = 0.0f;
            int t = 0;
            for (int i = 0; i < g.KH; ++i) {
                const int ih = oh * g.SH - g.PH + i * g.DH;
                const bool row_in = static_cast<unsigned>(ih) < static_cast<unsigned>(g.H);
                const long long row = (plane + ih) * g.W;
                for (int j = 0; j < g.KW; ++j, ++t) {
                    const int iw = ow * g.SW - g.PW + j * g.DW;
                    int xi = pad_index;
                    if (row_in && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W)) xi = index_of<DT>(x, row + iw);
                    int bits;
                    if (SMEM) {
                        bits = s_col[(t << 8) + xi];
                    } else {
                        const int flat = (static_cast<int>(wc[t]) << 8) | xi;
                        if (cls == LUT_I16) bits = static_cast<int>(__ldg(img->tabT16 + flat));
                        else if (cls == LUT_U16) bits = static_cast<int>(static_cast<uint16_t>(__ldg(img->tabT16 + flat)));
                        else bits = __float_as_int(__ldg(img->tabT32 + flat));
                    }
                    if (cls == LUT_F32) fsum += __int_as_float(bits);
                    else isum += bits;
                }
            }
            yn[l] = (cls == LUT_F32) ? fsum : static_cast<float>(isum);
        }
    }
}

// ---- backward: gradient with respect to the quantised image ---------------------------------------------------------
// One thread per image pixel; the channel's mapped weights dx[w(c, t)] (times the optional per-channel scale) sit
// in shared memory.  grid (C, slices).
__global__ void __launch_bounds__(kDwThreads) dwconv_grad_x_kernel(const float* __restrict__ go, const uint8_t* __restrict__ widx,
                                                                   const float* __restrict__ dx, const float* __restrict__ gs,
                                                                   float* __restrict__ gx, int N, ConvGeom g, long long chunk)
{
    __shared__ float s_w[kDwMaxTaps];
    const int c = blockIdx.x;
    const int taps = g.KH * g.KW;
    const float scale = gs != nullptr ? __ldg(gs + c) : 1.0f;
    for (int t = threadIdx.x; t < taps; t += blockDim.x)
        s_w[t] = __ldg(dx + widx[static_cast<long long>(c) * taps + t]) * scale;
    __syncthreads();
    const long long HW = static_cast<long long>(g.H) * g.W;
    const long long P = static_cast<long long>(N) * HW;
    const long long L = static_cast<long long>(g.OH) * g.OW;
    const long long p_end = min(P, (static_cast<long long>(blockIdx.y) + 1) * chunk);
    for (long long p = static_cast<long long>(blockIdx.y) * chunk + threadIdx.x; p < p_end; p += blockDim.x) {
        const long long n = p / HW;
        const int hw = static_cast<int>(p - n * HW);
        const int h = hw / g.W, w = hw - h * g.W;
        const float* gon = go + (n * g.C + c) * L;
        float acc = 0.0f;
        for (int i = 0; i < g.KH; ++i) {
            const int th = h + g.PH - i * g.DH;
            if (th < 0 || th % g.SH != 0) continue;
            const int oh = th / g.SH;
            if (oh >= g.OH) continue;
            for (int j = 0; j < g.KW; ++j) {
                const int tw = w + g.PW - j * g.DW;
                if (tw < 0 || tw % g.SW != 0) continue;
                const int ow = tw / g.SW;
                if (ow >= g.OW) continue;
                acc = fmaf(__ldg(gon + oh * g.OW + ow), s_w[i * g.KW + j], acc);
            }
        }
        gx[(n * g.C + c) * HW + hw] = acc;
    }
}

// ---- backward: gradient with respect to the quantised weights ---------------------------------------------------------
// grid (C, slices): block (c, s) sums its slice of the channel's output pixels for every tap, then adds the kh*kw
// block sums to grad_w[c, :] (atomics only across slices; one slice gives a deterministic result).
template <int DT>
__global__ void __launch_bounds__(kDwThreads) dwconv_grad_w_kernel(const float* __restrict__ go, const void* __restrict__ x,
                                                                   const float* __restrict__ dw, const float* __restrict__ gs,
                                                                   float* __restrict__ gw, int N, ConvGeom g, int pad_index,
                                                                   long long chunk)
{
    __shared__ float s_dw[257];
    __shared__ float s_part[kDwThreads / 32];
    for (int i = threadIdx.x; i < 257; i += blockDim.x) s_dw[i] = __ldg(dw + min(i, pad_index == 256 ? 256 : 255));
    __syncthreads();
    const int c = blockIdx.x;
    const int taps = g.KH * g.KW;
    const long long L = static_cast<long long>(g.OH) * g.OW;
    const long long P = static_cast<long long>(N) * L;
    const long long p_beg = static_cast<long long>(blockIdx.y) * chunk;
    const long long p_end = min(P, p_beg + chunk);
    const float scale = gs != nullptr ? __ldg(gs + c) : 1.0f;
    int t = 0;
    for (int i = 0; i < g.KH; ++i) {
        for (int j = 0; j < g.KW; ++j, ++t) {
            float acc = 0.0f;
            for (long long p = p_beg + threadIdx.x; p < p_end; p += blockDim.x) {
                const long long n = p / L;
                const int l = static_cast<int>(p - n * L);
                const int oh = l / g.OW, ow = l - oh * g.OW;
                const int ih = oh * g.SH - g.PH + i * g.DH;
                const int iw = ow * g.SW - g.PW + j * g.DW;
                int xi = pad_index;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
                    xi = index_of<DT>(x, ((n * g.C + c) * g.H + ih) * g.W + iw);
                acc = fmaf(__ldg(go + (n * g.C + c) * L + l), s_dw[xi], acc);
            }
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
            if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                float s = 0.0f;
                for (int k = 0; k < kDwThreads / 32; ++k) s += s_part[k];
                s *= scale;
                if (gridDim.y == 1) gw[static_cast<long long>(c) * taps + t] = s;
                else atomicAdd(gw + static_cast<long long>(c) * taps + t, s);
            }
            __syncthreads();
        }
    }
}

__global__ void dw_zero_kernel(float* p, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = 0.0f;
}

// slices per channel so that the grid has a few blocks per SM, each with at least a few thousand pixels
static void dw_grid(long long pixels, int C, int* slices, long long* chunk)
{
    const long long want = (4LL * sm_count() + C - 1) / (C > 0 ? C : 1);
    long long s = want < 1 ? 1 : want;
    const long long most = (pixels + 2047) / 2048;
    if (s > most) s = most;
    if (s < 1) s = 1;
    if (s > 65535) s = 65535;
    *chunk = (pixels + s - 1) / s;
    *slices = static_cast<int>((pixels + *chunk - 1) / *chunk);
}

template <int DT>
static void launch_dw_fwd(const void* x, const uint8_t* widx, const LutImage* img, float* y, int N, const ConvGeom& g,
                          int pad_index, cudaStream_t s)
{
    int slices;
    long long chunk;
    dw_grid(static_cast<long long>(N) * g.OH * g.OW, g.C, &slices, &chunk);
    const dim3 grid(g.C, slices);
    const int taps = g.KH * g.KW;
    if (taps <= kDwMaxTaps) {
        const size_t smem = static_cast<size_t>(taps) * 256 * 4;
        if (smem > 48 * 1024) cudaFuncSetAttribute(dwconv_fwd_kernel<DT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDwMaxTaps * 1024);
        dwconv_fwd_kernel<DT, true><<<grid, kDwThreads, smem, s>>>(x, widx, img, y, N, g, pad_index, chunk);
    } else {
        dwconv_fwd_kernel<DT, false><<<grid, kDwThreads, 0, s>>>(x, widx, img, y, N, g, pad_index, chunk);
    }
}

}  // namespace atb

using namespace atb;

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
    ATB_REQUIRE(C <= 2147483647 / (kh * kw), "too many channels");
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const LutImage* img = static_cast<const LutImage*>(lut_image);
    switch (dtype) {
        case ATB_F32: launch_dw_fwd<ATB_F32>(x, widx, img, y, N, g, pad_index, s); break;
        case ATB_I8: launch_dw_fwd<ATB_I8>(x, widx, img, y, N, g, pad_index, s); break;
        case ATB_U8: launch_dw_fwd<ATB_U8>(x, widx, img, y, N, g, pad_index, s); break;
        default: return fail_invalid("dtype must be ATB_F32, ATB_I8 or ATB_U8");
    }
    return check_launch("dwconv_fwd_kernel");
}

extern "C" int atb_lut_dwconv_bwd(const float* go, const void* x, int dtype, const uint8_t* widx,
                                  const float* dx, const float* dw_tab, const float* go_scale,
                                  float* grad_x, float* grad_w,
                                  int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
                                  int dh, int dw, int pad_index, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0, "negative dimension");
    ATB_REQUIRE(dtype == ATB_F32 || dtype == ATB_I8 || dtype == ATB_U8, "dtype must be ATB_F32, ATB_I8 or ATB_U8");
    ATB_REQUIRE(pad_index >= 0 && pad_index <= 256, "pad_index out of range");
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw, &OH, &OW), "conv geometry yields empty output");
    ATB_REQUIRE(kh * kw <= kDwMaxTaps, "depthwise backward supports windows of up to 49 taps");
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (C == 0) return ATB_OK;
    int rc = ATB_OK;
    if (grad_x != nullptr && static_cast<long long>(N) * H * W > 0) {
        ATB_REQUIRE(go && widx && dx, "null pointer");
        int slices;
        long long chunk;
        dw_grid(static_cast<long long>(N) * H * W, C, &slices, &chunk);
        dwconv_grad_x_kernel<<<dim3(C, slices), kDwThreads, 0, s>>>(go, widx, dx, go_scale, grad_x, N, g, chunk);
        rc = check_launch("dwconv_grad_x_kernel");
        if (rc != ATB_OK) return rc;
    }
    if (grad_w != nullptr) {
        const long long numel = static_cast<long long>(C) * kh * kw;
        int slices;
        long long chunk;
        dw_grid(static_cast<long long>(N) * OH * OW, C, &slices, &chunk);
        if (slices > 1 || static_cast<long long>(N) * OH * OW == 0) {
            dw_zero_kernel<<<grid_for(numel, 256, 1024), 256, 0, s>>>(grad_w, numel);
            rc = check_launch("dw_zero_kernel");
            if (rc != ATB_OK) return rc;
        }
        if (static_cast<long long>(N) * OH * OW > 0) {
            ATB_REQUIRE(go && x && dw_tab, "null pointer");
            const dim3 grid(C, slices);
            switch (dtype) {
                case ATB_F32: dwconv_grad_w_kernel<ATB_F32><<<grid, kDwThreads, 0, s>>>(go, x, dw_tab, go_scale, grad_w, N, g, pad_index, chunk); break;
                case ATB_I8: dwconv_grad_w_kernel<ATB_I8><<<grid, kDwThreads, 0, s>>>(go, x, dw_tab, go_scale, grad_w, N, g, pad_index, chunk); break;
                default: dwconv_grad_w_kernel<ATB_U8><<<grid, kDwThreads, 0, s>>>(go, x, dw_tab, go_scale, grad_w, N, g, pad_index, chunk); break;
            }
            rc = check_launch("dwconv_grad_w_kernel");
        }
    }
    return rc;
}
