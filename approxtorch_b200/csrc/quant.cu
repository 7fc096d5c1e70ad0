// Fake-quantisation, statistics and operand prepasses: HBM-bound streaming kernels.
// Each element is read once and written once with 16-byte accesses where the pointers allow;
// grids are sized from the SM count and stride over the tensor.
//
// Arithmetic contract (approxtorch/backend/csrc/claude/quantization.cu:54-75):
//   s = max(scale, 1e-12); v = x / s (+ z) with an IEEE fp32 division; mask = qmin <= v <= qmax on
//   the pre-round value; q = clamp(nearbyint(v), qmin, qmax) with round-half-even; NaN stays NaN in q.
#include "common.cuh"

namespace atb {

constexpr int kThreads = 256;

static int stream_grid(long long work_items)
{
    return grid_for(work_items, kThreads, 16 * sm_count());
}

// Grid-stride loop over n 16-byte (or 4-byte) vectors with FOUR loads per thread in flight before the first is
// consumed: a pass that moves one vector per iteration is bound by the load latency at about half of the HBM
// bandwidth.  The operands are read once, so they are loaded with the streaming (evict-first) hint.
template <class V, class F>
__device__ __forceinline__ void stream4(const V* __restrict__ src, long long n, F&& f)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
        const V v0 = __ldcs(src + i), v1 = __ldcs(src + i + stride), v2 = __ldcs(src + i + 2 * stride),
                v3 = __ldcs(src + i + 3 * stride);
        f(i, v0); f(i + stride, v1); f(i + 2 * stride, v2); f(i + 3 * stride, v3);
    }
    for (; i < n; i += stride) f(i, __ldcs(src + i));
}
// the same with a second operand stream read at the same index
template <class V, class W, class F>
__device__ __forceinline__ void stream4(const V* __restrict__ src, const W* __restrict__ src2, long long n, F&& f)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
        const V v0 = __ldcs(src + i), v1 = __ldcs(src + i + stride), v2 = __ldcs(src + i + 2 * stride),
                v3 = __ldcs(src + i + 3 * stride);
        const W w0 = __ldcs(src2 + i), w1 = __ldcs(src2 + i + stride), w2 = __ldcs(src2 + i + 2 * stride),
                w3 = __ldcs(src2 + i + 3 * stride);
        f(i, v0, w0); f(i + stride, v1, w1); f(i + 2 * stride, v2, w2); f(i + 3 * stride, v3, w3);
    }
    for (; i < n; i += stride) f(i, __ldcs(src + i), __ldcs(src2 + i));
}

__device__ __forceinline__ float fq_value(float x, float s, float z, float qmin, float qmax, bool& inside)
{
    const float v = x / s + z;     // z == 0 for the symmetric form; x/s + 0.0f == x/s bit for bit except -0 -> +0
    inside = (v >= qmin) && (v <= qmax);
    float r = nearbyintf(v);
    r = r < qmin ? qmin : r;
    r = r > qmax ? qmax : r;
    return r;
}

__device__ __forceinline__ float fq_value_sym(float x, float s, float qmin, float qmax, bool& inside)
{
    const float v = x / s;
    inside = (v >= qmin) && (v <= qmax);
    float r = nearbyintf(v);
    r = r < qmin ? qmin : r;
    r = r > qmax ? qmax : r;
    return r;
}

// ---- fp32 q + bool mask (the reference operator's outputs) ----------------------------------
template <bool VEC, bool ASYM>
__global__ void __launch_bounds__(kThreads, 4) fakequant_fwd_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                                     const float* __restrict__ zero, float* __restrict__ q,
                                     uint8_t* __restrict__ mask, long long numel, float qmin, float qmax)
{
    const float s = fmaxf(__ldg(scale), 1e-12f);
    const float z = ASYM ? __ldg(zero) : 0.0f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = VEC ? (numel >> 2) : 0;
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        float4* q4 = reinterpret_cast<float4*>(q);
        uchar4* m4 = reinterpret_cast<uchar4*>(mask);
        stream4(x4, n4, [&](long long i, const float4 v) {
            bool a, b, c, d;
            float4 r;
            if (ASYM) {
                r.x = fq_value(v.x, s, z, qmin, qmax, a); r.y = fq_value(v.y, s, z, qmin, qmax, b);
                r.z = fq_value(v.z, s, z, qmin, qmax, c); r.w = fq_value(v.w, s, z, qmin, qmax, d);
            } else {
                r.x = fq_value_sym(v.x, s, qmin, qmax, a); r.y = fq_value_sym(v.y, s, qmin, qmax, b);
                r.z = fq_value_sym(v.z, s, qmin, qmax, c); r.w = fq_value_sym(v.w, s, qmin, qmax, d);
            }
            q4[i] = r;
            m4[i] = make_uchar4(a, b, c, d);
        });
    }
    for (long long i = (n4 << 2) + t0; i < numel; i += stride) {
        bool a;
        q[i] = ASYM ? fq_value(x[i], s, z, qmin, qmax, a) : fq_value_sym(x[i], s, qmin, qmax, a);
        mask[i] = a;
    }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads, 4) fakequant_bwd_kernel(const float* __restrict__ go, const uint8_t* __restrict__ mask,
                                     const float* __restrict__ scale, float* __restrict__ gx, long long numel)
{
    const float s = fmaxf(__ldg(scale), 1e-12f);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = VEC ? (numel >> 2) : 0;
    if (VEC) {
        const float4* g4 = reinterpret_cast<const float4*>(go);
        const uchar4* m4 = reinterpret_cast<const uchar4*>(mask);
        float4* o4 = reinterpret_cast<float4*>(gx);
        stream4(g4, m4, n4, [&](long long i, const float4 g, const uchar4 m) {
            float4 r;
            r.x = (m.x ? g.x : 0.0f) / s; r.y = (m.y ? g.y : 0.0f) / s;
            r.z = (m.z ? g.z : 0.0f) / s; r.w = (m.w ? g.w : 0.0f) / s;
            o4[i] = r;
        });
    }
    for (long long i = (n4 << 2) + t0; i < numel; i += stride) gx[i] = (mask[i] ? go[i] : 0.0f) / s;
}

// ---- fused form: 1-byte quantised image + mask -------------------------------------------------
// symmetric: int8 value q; asymmetric: uint8 index q (q is already in [0,255])
template <bool VEC, bool ASYM, bool MASK>
__global__ void __launch_bounds__(kThreads, 4) quantize_image_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                                      const float* __restrict__ zero, uint8_t* __restrict__ q8,
                                      uint8_t* __restrict__ mask, long long numel, float qmin, float qmax)
{
    const float s = fmaxf(__ldg(scale), 1e-12f);
    const float z = ASYM ? __ldg(zero) : 0.0f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = VEC ? (numel >> 2) : 0;
    auto one = [&](float xv, bool& inside) -> uint8_t {
        const float r = ASYM ? fq_value(xv, s, z, qmin, qmax, inside) : fq_value_sym(xv, s, qmin, qmax, inside);
        // NaN has no 8-bit image: it becomes quantised zero (the fp32 operator would carry NaN on)
        const int qi = (r == r) ? static_cast<int>(r) : (ASYM ? static_cast<int>(z) : 0);
        return static_cast<uint8_t>(qi);      // two's complement low byte: int8 value or uint8 index
    };
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        uchar4* o4 = reinterpret_cast<uchar4*>(q8);
        uchar4* m4 = reinterpret_cast<uchar4*>(mask);
        stream4(x4, n4, [&](long long i, const float4 v) {
            bool a, b, c, d;
            uchar4 r;
            r.x = one(v.x, a); r.y = one(v.y, b); r.z = one(v.z, c); r.w = one(v.w, d);
            o4[i] = r;
            if (MASK) m4[i] = make_uchar4(a, b, c, d);
        });
    }
    for (long long i = (n4 << 2) + t0; i < numel; i += stride) {
        bool a;
        q8[i] = one(x[i], a);
        if (MASK) mask[i] = a;
    }
}

// ---- per-output-channel weight quantisation: one block per channel -------------------------------
__global__ void quantize_weight_kernel(const float* __restrict__ w, const float* __restrict__ scale,
                                       const float* __restrict__ zero, float qmin, float qmax, int index_offset,
                                       int inner, uint8_t* __restrict__ widx, uint8_t* __restrict__ mask,
                                       float* __restrict__ q, int* __restrict__ wsum)
{
    const int o = blockIdx.x;
    const float s = fmaxf(__ldg(scale + o), 1e-12f);
    const bool asym = zero != nullptr;
    const float z = asym ? __ldg(zero + o) : 0.0f;
    const long long base = static_cast<long long>(o) * inner;
    int local = 0;
    for (int i = threadIdx.x; i < inner; i += blockDim.x) {
        bool inside;
        const float r = asym ? fq_value(w[base + i], s, z, qmin, qmax, inside)
                             : fq_value_sym(w[base + i], s, qmin, qmax, inside);
        int idx = ((r == r) ? static_cast<int>(r) : 0) + index_offset;
        idx = max(0, min(255, idx));
        widx[base + i] = static_cast<uint8_t>(idx);
        if (mask != nullptr) mask[base + i] = inside;
        if (q != nullptr) q[base + i] = r;
        local += idx;
    }
    if (wsum != nullptr) {
        __shared__ int part[32];
        for (int off = 16; off > 0; off >>= 1) local += __shfl_down_sync(0xffffffffu, local, off);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = local;
        __syncthreads();
        if (threadIdx.x < 32) {
            int v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0;
            for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
            if (threadIdx.x == 0) wsum[o] = v;
        }
    }
}

// ---- statistics -------------------------------------------------------------------------------------
__global__ void stats_init_kernel(float* result)
{
    result[0] = 0.0f;
    result[1] = __int_as_float(0x7f800000);    // +inf
    result[2] = __int_as_float(0xff800000);    // -inf
}

// Float min / max through integer atomics.  Non-negative floats order like signed ints, negative floats order
// in reverse like unsigned ints, so the branch is taken on the SIGN BIT (-0.0 belongs with the negatives; a
// comparison with 0.0f would send it down the signed path as INT_MIN and wipe out a stored negative minimum).
__device__ __forceinline__ void atomic_min_float(float* addr, float v)
{
    if (__float_as_int(v) >= 0) atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
    else atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_max_float(float* addr, float v)
{
    if (__float_as_int(v) >= 0) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
// NaN markers that no later atomic of the two functions above can displace: the minimum slot takes the NaN
// with the sign bit set (largest unsigned, negative as an int), the maximum slot the positive NaN (largest int,
// smaller as an unsigned than any negative float).
__device__ __forceinline__ void atomic_min_nan(float* addr) { atomicMax(reinterpret_cast<unsigned int*>(addr), 0xffc00000u); }
__device__ __forceinline__ void atomic_max_nan(float* addr) { atomicMax(reinterpret_cast<int*>(addr), 0x7fc00000); }

// result[0] = max|x|, result[1] = min, result[2] = max; a NaN anywhere makes all three NaN, as torch's
// max / amin / amax do
template <bool VEC, bool MINMAX>
__global__ void stats_kernel(const float* __restrict__ x, long long numel, float* __restrict__ result)
{
    float am = 0.0f, mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
    auto take = [&](float v) {
        const float a = fabsf(v);
        am = (a > am || a != a) ? a : am;
        if (MINMAX) { mn = (v < mn || v != v) ? v : mn; mx = (v > mx || v != v) ? v : mx; }
    };
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = VEC ? (numel >> 2) : 0;
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        stream4(x4, n4, [&](long long, const float4 v) { take(v.x); take(v.y); take(v.z); take(v.w); });
    }
    for (long long i = (n4 << 2) + t0; i < numel; i += stride) take(x[i]);
    for (int off = 16; off > 0; off >>= 1) {
        const float o = __shfl_down_sync(0xffffffffu, am, off);
        am = (o > am || o != o) ? o : am;
        if (MINMAX) {
            const float on = __shfl_down_sync(0xffffffffu, mn, off), ox = __shfl_down_sync(0xffffffffu, mx, off);
            mn = (on < mn || on != on) ? on : mn;
            mx = (ox > mx || ox != ox) ? ox : mx;
        }
    }
    // one atomic per block and statistic: the warps' results meet in shared memory first (thousands of atomics on
    // the same three words would queue up behind one another at the end of the pass)
    __shared__ float s_am[32], s_mn[32], s_mx[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    if (lane == 0) { s_am[warp] = am; if (MINMAX) { s_mn[warp] = mn; s_mx[warp] = mx; } }
    __syncthreads();
    if (warp == 0) {
        am = lane < nwarps ? s_am[lane] : 0.0f;
        if (MINMAX) {
            mn = lane < nwarps ? s_mn[lane] : __int_as_float(0x7f800000);
            mx = lane < nwarps ? s_mx[lane] : __int_as_float(0xff800000);
        }
        for (int off = 16; off > 0; off >>= 1) {
            const float o = __shfl_down_sync(0xffffffffu, am, off);
            am = (o > am || o != o) ? o : am;
            if (MINMAX) {
                const float on = __shfl_down_sync(0xffffffffu, mn, off), ox = __shfl_down_sync(0xffffffffu, mx, off);
                mn = (on < mn || on != on) ? on : mn;
                mx = (ox > mx || ox != ox) ? ox : mx;
            }
        }
        if (lane == 0) {
            atomicMax(reinterpret_cast<int*>(result), __float_as_int(am));   // |x| >= 0: int order == float order, NaN highest
            if (MINMAX) {
                if (mn != mn) atomic_min_nan(result + 1); else atomic_min_float(result + 1, mn);
                if (mx != mx) atomic_max_nan(result + 2); else atomic_max_float(result + 2, mx);
            }
        }
    }
}

// ---- operand prepasses ---------------------------------------------------------------------------------
template <bool VEC>
__global__ void quantize_u8_kernel(const float* __restrict__ in, uint8_t* __restrict__ out, long long numel, int offset)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n4 = VEC ? (numel >> 2) : 0;
    if (VEC) {
        const float4* in4 = reinterpret_cast<const float4*>(in);
        uchar4* out4 = reinterpret_cast<uchar4*>(out);
        stream4(in4, n4, [&](long long i, const float4 v) {
            out4[i] = make_uchar4(index_from_float(v.x, offset), index_from_float(v.y, offset),
                                  index_from_float(v.z, offset), index_from_float(v.w, offset));
        });
    }
    for (long long i = (n4 << 2) + t0; i < numel; i += stride) out[i] = index_from_float(in[i], offset);
}

// B[K,N] (element strides sk, sn) -> out[N,K]; 32x32 tile through shared memory
template <typename T>
__global__ void quantize_transpose_kernel(const T* __restrict__ b, uint8_t* __restrict__ out, int K, int N,
                                          long long sk, long long sn, int offset)
{
    __shared__ uint8_t tile[32][33];
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
        const int k = k0 + dy, n = n0 + threadIdx.x;
        if (k < K && n < N) {
            const T v = b[k * sk + n * sn];
            uint8_t idx;
            if constexpr (sizeof(T) == 4) idx = index_from_float(static_cast<float>(v), offset);
            else idx = static_cast<uint8_t>(v);
            tile[dy][threadIdx.x] = idx;
        }
    }
    __syncthreads();
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
        const int n = n0 + dy, k = k0 + threadIdx.x;
        if (n < N && k < K) out[static_cast<long long>(n) * K + k] = tile[threadIdx.x][dy];
    }
}

}  // namespace atb

using namespace atb;

extern "C" int atb_fakequant_fwd(const float* x, const float* scale, const float* zero_point, int qmin, int qmax,
                                 float* q, uint8_t* mask, long long numel, void* stream)
{
    ATB_REQUIRE(numel >= 0, "negative numel");
    if (numel == 0) return ATB_OK;
    ATB_REQUIRE(x && scale && q && mask, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = aligned_to(x, 16) && aligned_to(q, 16) && aligned_to(mask, 4);
    const int grid = stream_grid(vec ? numel / 4 + 1 : numel);
    const float lo = static_cast<float>(qmin), hi = static_cast<float>(qmax);
    if (zero_point) {
        if (vec) fakequant_fwd_kernel<true, true><<<grid, kThreads, 0, s>>>(x, scale, zero_point, q, mask, numel, lo, hi);
        else fakequant_fwd_kernel<false, true><<<grid, kThreads, 0, s>>>(x, scale, zero_point, q, mask, numel, lo, hi);
    } else {
        if (vec) fakequant_fwd_kernel<true, false><<<grid, kThreads, 0, s>>>(x, scale, nullptr, q, mask, numel, lo, hi);
        else fakequant_fwd_kernel<false, false><<<grid, kThreads, 0, s>>>(x, scale, nullptr, q, mask, numel, lo, hi);
    }
    return check_launch("fakequant_fwd_kernel");
}

extern "C" int atb_fakequant_bwd(const float* go, const uint8_t* mask, const float* scale, float* gx,
                                 long long numel, void* stream)
{
    ATB_REQUIRE(numel >= 0, "negative numel");
    if (numel == 0) return ATB_OK;
    ATB_REQUIRE(go && mask && scale && gx, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = aligned_to(go, 16) && aligned_to(gx, 16) && aligned_to(mask, 4);
    const int grid = stream_grid(vec ? numel / 4 + 1 : numel);
    if (vec) fakequant_bwd_kernel<true><<<grid, kThreads, 0, s>>>(go, mask, scale, gx, numel);
    else fakequant_bwd_kernel<false><<<grid, kThreads, 0, s>>>(go, mask, scale, gx, numel);
    return check_launch("fakequant_bwd_kernel");
}

template <bool VEC, bool ASYM>
static void launch_quantize_image(const float* x, const float* scale, const float* zero, uint8_t* q8, uint8_t* mask,
                                  long long numel, float lo, float hi, int grid, cudaStream_t s)
{
    if (mask) quantize_image_kernel<VEC, ASYM, true><<<grid, kThreads, 0, s>>>(x, scale, zero, q8, mask, numel, lo, hi);
    else quantize_image_kernel<VEC, ASYM, false><<<grid, kThreads, 0, s>>>(x, scale, zero, q8, nullptr, numel, lo, hi);
}

extern "C" int atb_quantize_image(const float* x, const float* scale, const float* zero_point, int qmin, int qmax,
                                  void* q8, uint8_t* mask, long long numel, void* stream)
{
    ATB_REQUIRE(numel >= 0, "negative numel");
    if (numel == 0) return ATB_OK;
    ATB_REQUIRE(x && scale && q8, "null pointer");
    if (zero_point) ATB_REQUIRE(qmin >= 0 && qmax <= 255, "asymmetric range must lie in [0, 255]");
    else ATB_REQUIRE(qmin >= -128 && qmax <= 127, "symmetric range must lie in [-128, 127]");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = aligned_to(x, 16) && aligned_to(q8, 4) && (mask == nullptr || aligned_to(mask, 4));
    const int grid = stream_grid(vec ? numel / 4 + 1 : numel);
    const float lo = static_cast<float>(qmin), hi = static_cast<float>(qmax);
    uint8_t* out = static_cast<uint8_t*>(q8);
    if (zero_point) {
        if (vec) launch_quantize_image<true, true>(x, scale, zero_point, out, mask, numel, lo, hi, grid, s);
        else launch_quantize_image<false, true>(x, scale, zero_point, out, mask, numel, lo, hi, grid, s);
    } else {
        if (vec) launch_quantize_image<true, false>(x, scale, nullptr, out, mask, numel, lo, hi, grid, s);
        else launch_quantize_image<false, false>(x, scale, nullptr, out, mask, numel, lo, hi, grid, s);
    }
    return check_launch("quantize_image_kernel");
}

extern "C" int atb_quantize_weight(const float* w, const float* scale, const float* zero_point, int qmin, int qmax,
                                   int index_offset, int O, int inner, uint8_t* widx, uint8_t* mask, float* q,
                                   int* wsum, void* stream)
{
    ATB_REQUIRE(O >= 0 && inner >= 0, "negative dimension");
    if (O == 0) return ATB_OK;
    ATB_REQUIRE(w && scale && widx, "null pointer");
    quantize_weight_kernel<<<O, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        w, scale, zero_point, static_cast<float>(qmin), static_cast<float>(qmax), index_offset, inner,
        widx, mask, q, wsum);
    return check_launch("quantize_weight_kernel");
}

extern "C" int atb_absmax(const float* x, long long numel, int want_minmax, float* result, void* stream)
{
    ATB_REQUIRE(numel >= 0 && result != nullptr, "bad arguments");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    stats_init_kernel<<<1, 1, 0, s>>>(result);
    int rc = check_launch("stats_init_kernel");
    if (rc != ATB_OK || numel == 0) return rc;
    ATB_REQUIRE(x != nullptr, "null pointer");
    const bool vec = aligned_to(x, 16);
    const int grid = grid_for(vec ? numel / 4 + 1 : numel, kThreads, 8 * sm_count());
    if (want_minmax) {
        if (vec) stats_kernel<true, true><<<grid, kThreads, 0, s>>>(x, numel, result);
        else stats_kernel<false, true><<<grid, kThreads, 0, s>>>(x, numel, result);
    } else {
        if (vec) stats_kernel<true, false><<<grid, kThreads, 0, s>>>(x, numel, result);
        else stats_kernel<false, false><<<grid, kThreads, 0, s>>>(x, numel, result);
    }
    return check_launch("stats_kernel");
}

extern "C" int atb_quantize_u8(const float* in, uint8_t* out, long long numel, int offset, void* stream)
{
    ATB_REQUIRE(numel >= 0, "negative numel");
    if (numel == 0) return ATB_OK;
    ATB_REQUIRE(in && out, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = aligned_to(in, 16) && aligned_to(out, 4);
    const int grid = stream_grid(vec ? numel / 4 + 1 : numel);
    if (vec) quantize_u8_kernel<true><<<grid, kThreads, 0, s>>>(in, out, numel, offset);
    else quantize_u8_kernel<false><<<grid, kThreads, 0, s>>>(in, out, numel, offset);
    return check_launch("quantize_u8_kernel");
}

extern "C" int atb_quantize_transpose_u8(const void* b, int dtype, int K, int N, long long stride_k,
                                         long long stride_n, int offset, uint8_t* out, void* stream)
{
    ATB_REQUIRE(K >= 0 && N >= 0, "negative dimension");
    ATB_REQUIRE(dtype == ATB_F32 || dtype == ATB_U8, "B must be fp32 values or uint8 indices");
    if (static_cast<long long>(K) * N == 0) return ATB_OK;
    ATB_REQUIRE(b && out, "null pointer");
    dim3 block(32, 8), grid(ceil_div(N, 32), ceil_div(K, 32));
    ATB_REQUIRE(grid.y <= 65535, "K too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ATB_F32)
        quantize_transpose_kernel<float><<<grid, block, 0, s>>>(static_cast<const float*>(b), out, K, N, stride_k, stride_n, offset);
    else
        quantize_transpose_kernel<uint8_t><<<grid, block, 0, s>>>(static_cast<const uint8_t*>(b), out, K, N, stride_k, stride_n, offset);
    return check_launch("quantize_transpose_kernel");
}
