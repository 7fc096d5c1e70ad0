// Library-wide runtime helpers: per-thread error text, device properties, LUT image preparation.
#include <stdarg.h>

#include "common.cuh"

namespace atb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// One thread per table entry.  Writes all four images and raises the two "not exact" flags
// (the flags were zeroed by the memset that precedes the launch).  Eligibility rules:
// approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:116-142.
__global__ void lut_prepare_kernel(const float* __restrict__ lut, LutImage* __restrict__ img)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;   // i = x * 256 + w
    const float v = lut[i];
    const float r = rintf(v);
    const bool is_int = (v == r);
    const bool i16_ok = is_int && (fabsf(v) <= 32767.0f);
    const bool u16_ok = is_int && (v >= 0.0f) && (v <= 65535.0f);
    if (!i16_ok) img->flags[0] = 1;
    if (!u16_ok) img->flags[1] = 1;
    const int16_t v16 = (i16_ok || u16_ok)
        ? static_cast<int16_t>(static_cast<uint16_t>(static_cast<int>(r))) : static_cast<int16_t>(0);
    const int t = ((i & 255) << 8) | (i >> 8);
    img->tab16[i] = v16;
    img->tab32[i] = v;
    img->tabT16[t] = v16;
    img->tabT32[t] = v;
    {
        const int xh = (i >> 8) >> 7, xl = (i >> 8) & 127;
        img->tabTP32[((i & 255) << 8) + (xh << 7) + ((xl & 31) << 2) + (xl >> 5)] = v;
    }
    const int xi = i >> 8, wi = i & 255;
    // pair i = xi & 127 = {x = i, x = i + 128} sits at word 4 * (i & 31) + (i >> 5) of row wi: a 16-byte load by
    // lane l then yields the pairs l, l + 32, l + 64, l + 96
    const int pair = xi & 127;
    img->tabTP16[(wi << 8) + (((pair & 31) << 2) + (pair >> 5)) * 2 + (xi >> 7)] = v16;
}

// Tables of the int16 class are looked up as unsigned entries carrying a +32768 bias (bit 15 flipped); the
// staged-lookup image is stored that way so that the GEMM blocks can copy it into shared memory untouched.
// Runs after lut_prepare_kernel on the same stream, when the class flags are final.
__global__ void lut_bias_kernel(LutImage* __restrict__ img)
{
    if (img->flags[0] != 0) return;                        // not the int16 class
    uint32_t* words = reinterpret_cast<uint32_t*>(img->tabTP16);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;   // 32768 words
    words[i] ^= 0x80008000u;
}

// Measurement aid: the rate at which an SM serves conflict-free 8-byte shared-memory loads, the instruction
// the LUT GEMM's lookups are made of.  Every thread issues `iters` x 8 independent loads whose 16 lanes per
// half-warp cover all 32 banks exactly once (consecutive 8-byte slots), adds the words up and stores the sum so
// that nothing can be optimised away.  Bank words served = threads x iters x 8 x 2.
__global__ void __launch_bounds__(1024, 1) shared_load_probe_kernel(const unsigned* __restrict__ seed, unsigned* __restrict__ out,
                                                                    int iters)
{
    __shared__ uint2 buf[4096];                            // 32 KB
    for (int i = threadIdx.x; i < 4096; i += blockDim.x) buf[i] = make_uint2(seed[i & 255], seed[(i + 1) & 255]);
    __syncthreads();
    unsigned a = 0u, b = 0u, idx = threadIdx.x;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint2 v = buf[(idx + 512u * u) & 4095u];
            a += v.x;
            b += v.y;
        }
        idx += 32u;
    }
    out[blockIdx.x * blockDim.x + threadIdx.x] = a + b;
}

}  // namespace atb

using namespace atb;

extern "C" int atb_probe_shared_load(const unsigned* seed256, unsigned* out, int blocks, int iters, void* stream)
{
    ATB_REQUIRE(seed256 != nullptr && out != nullptr && blocks > 0 && iters >= 0, "bad arguments");
    shared_load_probe_kernel<<<blocks, 1024, 0, static_cast<cudaStream_t>(stream)>>>(seed256, out, iters);
    return check_launch("shared_load_probe_kernel");
}

extern "C" const char* atb_last_error(void) { return g_error; }
extern "C" int atb_version(void) { return 100; }
extern "C" size_t atb_lut_image_bytes(void) { return sizeof(LutImage); }

extern "C" int atb_lut_prepare(const float* lut, void* image, void* stream)
{
    ATB_REQUIRE(lut != nullptr && image != nullptr, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(image, 0, sizeof(int) * 4, s);
    if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    ATB_REQUIRE(aligned_to(image, 16), "image must be 16-byte aligned");
    lut_prepare_kernel<<<256, 256, 0, s>>>(lut, static_cast<LutImage*>(image));
    int rc = check_launch("lut_prepare_kernel");
    if (rc != ATB_OK) return rc;
    lut_bias_kernel<<<128, 256, 0, s>>>(static_cast<LutImage*>(image));
    return check_launch("lut_bias_kernel");
}
