// STE / LRE image-space backward on the 5th-generation tensor cores (tcgen05.mma with the accumulator in TMEM).
//
//   grad_w[o,k] = gs[o] * sum_{p=(n,oh,ow)} go[p,o] * dw[idx(x[p,k]) or pad]           M = O,        N = C*kh*kw, reduce over pixels
//   grad_x[m,c] = sum_{r=(tap,o)} go[pixel m, tap, o] * gs[o] * (dx[widx[o,(c,tap)]] - wz[o])    M = image pixels, N = C
//
// Both are dense contractions whose operands are a table map (or a gather) of the saved 8-bit tensors, so nothing
// can be fetched by a tensor-map copy: the operand tiles are PRODUCED by the block's threads - gather, table map,
// split, store - straight into the shared-memory layout the tensor core reads, and one elected thread issues the
// MMAs.  fp32 accuracy (these gradients carry a rel-1e-5 bar, single-pass bf16 or tf32 cannot meet it) comes from
// splitting every fp32 operand value v into three bf16 terms hi + mid + lo (24 mantissa bits, exact) and issuing the
// six products hi*hi, hi*mid, mid*hi, mid*mid, hi*lo, lo*hi into one fp32 accumulator; when one operand is exactly
// representable in bf16 (the STE tables are the integers -128..127, minus an integer zero point) three suffice.
//
// Block = 128 x 128 output tile, 512 threads.  Per stage a 32-wide slice of the reduction: every thread produces
// eight elements of A and eight of B - the warp's lanes run along whichever axis is contiguous in memory, so each
// global load is one coalesced segment - and writes their bf16 terms into the K-major canonical layout without
// swizzle (8-row x 16-byte core matrices, k-groups 144 bytes apart so that a warp's stores fall into different
// banks, 8-row groups 576 bytes apart).  The raw values of the next slice are loaded right after this slice's have
// been stored, so their latency runs under the barrier and the MMA issue.  The writes are fenced for the
// asynchronous proxy, and after the block barrier thread 0 issues
// the stage's MMAs (two k=16 steps x 3 or 6 products) followed by a commit that arrives on the stage's mbarrier.
// Two stages: the tensor core works on one while the threads produce the other; a stage is rewritten only after its
// mbarrier reports the MMAs that read it complete (bounded wait: a block that gives up raises the status word and
// finishes without hanging).  Epilogue: each warp reads its 32 TMEM lanes x 32 columns (tcgen05.ld) and stores or
// atomically adds the tile.  grad_w splits the pixel axis over the grid (fp32 atomics into a zeroed output);
// grad_x runs per stride class and tap-major exactly like the SIMT kernel it replaces (grad_dense.cu), which stays
// as the general fallback and as the checker.
#include <cuda_bf16.h>

#include "common.cuh"

namespace atb {

constexpr int TcM = 128, TcN = 128, TcK = 32;
constexpr int TcThreads = 512;
// K-major canonical layout without swizzle: a core matrix is 8 rows x 16 bytes (8 bf16 of the reduction) stored
// contiguously; the k-groups of a row group lie TcLBO bytes apart and the 8-row groups TcSBO bytes apart.  144 =
// 128 + 16: the four k-groups a warp writes at once start 36 words apart, i.e. in different banks.
constexpr uint32_t TcLBO = 144;
constexpr uint32_t TcSBO = TcLBO * (TcK / 8);        // 576
constexpr int TcSplitBytes = 16 * TcSBO;             // one bf16 split of one 128-row operand tile: 9216
constexpr int TcStageBytes = 6 * TcSplitBytes;       // A hi/mid/lo, B hi/mid/lo: 55296
constexpr int TcSmemBytes = 2 * TcStageBytes;        // 110592
constexpr int TcMaxTaps = 128;

__device__ int g_tc_status = 0;                      // 1: a block gave up waiting for its MMAs

struct TcFastDiv {
    unsigned d, mul, shift;
};
static TcFastDiv tc_fastdiv(unsigned d)
{
    TcFastDiv f;
    f.d = d < 1 ? 1 : d;
    unsigned s = 0;
    while ((1ull << s) < f.d) ++s;
    f.shift = s;
    f.mul = static_cast<unsigned>((((1ull << s) - f.d) << 32) / f.d + 1);
    return f;
}
__device__ __forceinline__ unsigned tc_div(unsigned n, const TcFastDiv& f) { return (__umulhi(n, f.mul) + n) >> f.shift; }

// ---- shared-memory matrix descriptor (no swizzle) and instruction descriptor -----------------------------------------
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr)
{
    uint64_t d = static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(TcLBO >> 4) << 16;
    d |= static_cast<uint64_t>(TcSBO >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;             // descriptor version of sm_100
    return d;
}
// D fp32, A and B bf16, both K-major, M = 128, N = 128
constexpr uint32_t kTcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t tmem, uint64_t da, uint64_t db, bool accumulate)
{
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem), "l"(da), "l"(db), "r"(kTcIdesc), "r"(acc) : "memory");
}

__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity)
{
    for (int i = 0; i < (1 << 22); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// one fp32 value -> three bf16 terms, v = hi + mid + lo exactly
__device__ __forceinline__ void tc_split1(float v, uint16_t& hi, uint16_t& mid, uint16_t& lo)
{
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    const float r = v - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(r);
    const __nv_bfloat16 l = __float2bfloat16_rn(r - __bfloat162float(m));
    hi = __bfloat16_as_ushort(h); mid = __bfloat16_as_ushort(m); lo = __bfloat16_as_ushort(l);
}
// two fp32 values (consecutive reduction elements) -> three words of two bf16
__device__ __forceinline__ void tc_split2(float a, float b, uint32_t& hi, uint32_t& mid, uint32_t& lo)
{
    const __nv_bfloat162 ph = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&ph);
    const float ra = a - __uint_as_float(hi << 16), rb = b - __uint_as_float(hi & 0xffff0000u);
    const __nv_bfloat162 pm = __floats2bfloat162_rn(ra, rb);
    mid = *reinterpret_cast<const uint32_t*>(&pm);
    const float sa = ra - __uint_as_float(mid << 16), sb = rb - __uint_as_float(mid & 0xffff0000u);
    const __nv_bfloat162 pl = __floats2bfloat162_rn(sa, sb);
    lo = *reinterpret_cast<const uint32_t*>(&pl);
}

// eight fp32 values -> three rows of eight bf16 (hi, mid, lo), v = hi + mid + lo exactly
__device__ __forceinline__ void tc_split8(const float (&v)[8], uint4& hi, uint4& mid, uint4& lo)
{
    uint32_t h[4], m[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        const __nv_bfloat162 ph = __floats2bfloat162_rn(a, b);
        h[i] = *reinterpret_cast<const uint32_t*>(&ph);
        const float ra = a - __uint_as_float(h[i] << 16), rb = b - __uint_as_float(h[i] & 0xffff0000u);
        const __nv_bfloat162 pm = __floats2bfloat162_rn(ra, rb);
        m[i] = *reinterpret_cast<const uint32_t*>(&pm);
        const float sa = ra - __uint_as_float(m[i] << 16), sb = rb - __uint_as_float(m[i] & 0xffff0000u);
        const __nv_bfloat162 pl = __floats2bfloat162_rn(sa, sb);
        l[i] = *reinterpret_cast<const uint32_t*>(&pl);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    mid = make_uint4(m[0], m[1], m[2], m[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// ---- problem: grad_w ----------------------------------------------------------------------------------------------------
// C[o, k] = gs[o] * sum_p go[n,o,l] * dw[idx(x[n,c,ih,iw]) or pad];  rows of A: o, rows of B: k = (c,i,j); reduction: p.
// Producer mapping: the 32 lanes of a warp are the 32 consecutive pixels of the slice (contiguous in go and, for a
// stride-1 window, in x), warp w produces rows w, w + 16, ... of both tiles: every global load is one coalesced
// segment per row, every element is stored as three 2-byte terms.
template <int XDT>
struct TcGradW {
    const float* go; const void* x; const float* dw; const float* gs; float* gw;
    int O, K, pad_index, Nb; long long P; ConvGeom g;
    TcFastDiv divL, divOW, divKK, divKW;
    static constexpr bool kAtomic = true;
    const float* tab;                   // dw (257 entries) in shared memory
    // thread state: the 8 rows this thread produces (row = warp + 16 i)
    int o_off[8];                       // o * L, or -1
    int x_koff[8];                      // tap offset from the window origin
    int k_dhw[8];                       // (i*DH - PH) << 16 | (j*DW - PW) & 0xffff; INT_MIN: no such tap
    uint32_t soff[8];                   // byte offset of (row, lane) inside a split tile
    __device__ int M() const { return O; }
    __device__ int N() const { return K; }
    __device__ void setup(int z, int nz, int& rbeg, int& rend)
    {
        __shared__ float s_tab[257];
        for (int i = threadIdx.x; i < 257; i += blockDim.x) s_tab[i] = __ldg(dw + (i < 256 || pad_index == 256 ? i : 255));
        __syncthreads();
        tab = s_tab;
        const long long per = ((P + nz - 1) / nz + TcK - 1) / TcK * TcK;
        const long long b0 = per * z;
        rbeg = static_cast<int>(b0 < P ? b0 : P);
        rend = static_cast<int>(b0 + per < P ? b0 + per : P);
    }
    __device__ void prep(int warp, int lane, int m0, int n0)
    {
        const int L = g.OH * g.OW;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = warp + 16 * i;
            const int o = m0 + row;
            o_off[i] = o < O ? o * L : -1;
            const int k = n0 + row;
            k_dhw[i] = INT_MIN; x_koff[i] = 0;
            if (k < K) {
                const unsigned c = tc_div(k, divKK);
                const unsigned ij = k - c * (g.KH * g.KW);
                const unsigned ti = tc_div(ij, divKW);
                const unsigned tj = ij - ti * g.KW;
                const int dh = static_cast<int>(ti) * g.DH - g.PH, dw_ = static_cast<int>(tj) * g.DW - g.PW;
                k_dhw[i] = (dh << 16) | (dw_ & 0xffff);
                x_koff[i] = (static_cast<int>(c) * g.H + dh) * g.W + dw_;
            }
            soff[i] = static_cast<uint32_t>(row >> 3) * TcSBO + static_cast<uint32_t>(lane >> 3) * TcLBO +
                      static_cast<uint32_t>(row & 7) * 16u + static_cast<uint32_t>(lane & 7) * 2u;
        }
    }
    // raw values of the slice starting at reduction index r0: this lane's pixel is r0 + lane
    __device__ void load(int r0, int rend, int warp, int lane, float (&va)[8], float (&vb)[8]) const
    {
        const int L = g.OH * g.OW;
        const int p = r0 + lane;
        const bool live = p < rend;
        const unsigned n = tc_div(live ? p : 0, divL);
        const int l = (live ? p : 0) - static_cast<int>(n) * L;
        const int oh = static_cast<int>(tc_div(l, divOW));
        const int ow = l - oh * g.OW;
        const float* go_p = go + static_cast<int>(n) * O * L + l;
        const int x_p = (static_cast<int>(n) * g.C * g.H + oh * g.SH) * g.W + ow * g.SW;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            va[i] = (live && o_off[i] >= 0) ? __ldg(go_p + o_off[i]) : 0.0f;
            float b = 0.0f;
            if (live && k_dhw[i] != INT_MIN) {
                const int ih = oh * g.SH + (k_dhw[i] >> 16), iw = ow * g.SW + static_cast<short>(k_dhw[i] & 0xffff);
                int idx = pad_index;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
                    idx = index_of<XDT>(x, x_p + x_koff[i]);
                b = tab[idx];
            }
            vb[i] = b;
        }
    }
    template <bool EXACT_B>
    __device__ void store(uint8_t* stage, const float (&va)[8], const float (&vb)[8]) const
    {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint16_t hi, mid, lo;
            tc_split1(va[i], hi, mid, lo);
            *reinterpret_cast<uint16_t*>(stage + soff[i]) = hi;
            *reinterpret_cast<uint16_t*>(stage + TcSplitBytes + soff[i]) = mid;
            *reinterpret_cast<uint16_t*>(stage + 2 * TcSplitBytes + soff[i]) = lo;
            if (EXACT_B) {
                *reinterpret_cast<uint16_t*>(stage + 3 * TcSplitBytes + soff[i]) = __bfloat16_as_ushort(__float2bfloat16_rn(vb[i]));
            } else {
                tc_split1(vb[i], hi, mid, lo);
                *reinterpret_cast<uint16_t*>(stage + 3 * TcSplitBytes + soff[i]) = hi;
                *reinterpret_cast<uint16_t*>(stage + 4 * TcSplitBytes + soff[i]) = mid;
                *reinterpret_cast<uint16_t*>(stage + 5 * TcSplitBytes + soff[i]) = lo;
            }
        }
    }
    __device__ void finish(int o, int k, float v) const
    {
        if (gs != nullptr) v *= __ldg(gs + o);
        atomicAdd(gw + o * K + k, v);
    }
};

// ---- problem: grad_x, per stride class, tap-major ---------------------------------------------------------------------------
// Pixels are grouped by class (a, b) = ((h + PH) % SH, (w + PW) % SW) = blockIdx.z; a class only receives from the
// taps with (a - i*DH) % SH == 0 and (b - j*DW) % SW == 0.  C[m, c] with m the class's pixels; reduction index
// r = tap * O8 + o (O8 = O rounded up to 8).
// Producer mapping: the 32 lanes of a warp are 32 consecutive rows (pixels of A, contiguous in go; channels of B),
// warp w produces the two adjacent reduction elements 2w, 2w + 1 of the slice for the four 32-row groups: every go
// load is one coalesced segment, every store is one 32-bit word holding both elements.
struct TcGradX {
    const float* go; const uint8_t* widx; const float* dx; const float* gs; const float* wz; float* gx;
    int Nb, O, K, O8; ConvGeom g;
    TcFastDiv divSH, divSW;
    const uint8_t* xmask; const float* xscale;      // optional: fake-quant backward (mask ? v : 0) / max(scale, 1e-12) in the store
    static constexpr bool kAtomic = false;
    // block state
    int Mc, Hc, Wc, h0, w0, ntaps;
    const int* tap_dh; const int* tap_dw; const int* tap_ij;
    const float* tab;                   // dx in shared memory
    // thread state: four rows (32 rg + lane)
    int hp[4], wp[4], go_n[4], ckk[4];
    uint32_t soff[4];
    __device__ int M() const { return Mc; }
    __device__ int N() const { return g.C; }
    __device__ void setup(int z, int, int& rbeg, int& rend)
    {
        __shared__ int s_dh[TcMaxTaps], s_dw[TcMaxTaps], s_ij[TcMaxTaps], s_n;
        __shared__ float s_tab[256];
        for (int i = threadIdx.x; i < 256; i += blockDim.x) s_tab[i] = __ldg(dx + i);
        tab = s_tab;
        const int a = z / g.SW, b = z - a * g.SW;
        h0 = ((a - g.PH) % g.SH + g.SH) % g.SH;
        w0 = ((b - g.PW) % g.SW + g.SW) % g.SW;
        Hc = h0 < g.H ? (g.H - h0 + g.SH - 1) / g.SH : 0;
        Wc = w0 < g.W ? (g.W - w0 + g.SW - 1) / g.SW : 0;
        Mc = Nb * Hc * Wc;
        if (threadIdx.x == 0) {
            int n = 0;
            for (int i = 0; i < g.KH; ++i) {
                if (((a - i * g.DH) % g.SH + g.SH) % g.SH != 0) continue;
                for (int j = 0; j < g.KW; ++j) {
                    if (((b - j * g.DW) % g.SW + g.SW) % g.SW != 0) continue;
                    s_dh[n] = i * g.DH; s_dw[n] = j * g.DW; s_ij[n] = i * g.KW + j; ++n;
                }
            }
            s_n = n;
        }
        __syncthreads();
        ntaps = s_n;
        tap_dh = s_dh; tap_dw = s_dw; tap_ij = s_ij;
        rbeg = 0; rend = ntaps * O8;
    }
    __device__ void pixel_of(int m, int& n, int& h, int& w) const
    {
        const int hw = Hc * Wc;
        n = m / hw;
        const int rem = m - n * hw;
        const int t = rem / Wc;
        h = h0 + g.SH * t;
        w = w0 + g.SW * (rem - t * Wc);
    }
    __device__ void prep(int warp, int lane, int m0, int n0)
    {
#pragma unroll
        for (int rg = 0; rg < 4; ++rg) {
            const int row = 32 * rg + lane;
            const int m = m0 + row;
            hp[rg] = wp[rg] = -(1 << 28);
            go_n[rg] = 0;
            if (m < Mc) {
                int n, h, w;
                pixel_of(m, n, h, w);
                hp[rg] = h + g.PH; wp[rg] = w + g.PW;
                go_n[rg] = n * O * g.OH * g.OW;
            }
            const int c = n0 + row;
            ckk[rg] = c < g.C ? c * (g.KH * g.KW) : -1;
            soff[rg] = static_cast<uint32_t>(row >> 3) * TcSBO + static_cast<uint32_t>((2 * warp) >> 3) * TcLBO +
                       static_cast<uint32_t>(row & 7) * 16u + static_cast<uint32_t>((2 * warp) & 7) * 2u;
        }
    }
    // slot 2 rg + e: row group rg, reduction element r0 + 2 warp + e
    __device__ void load(int r0, int rend, int warp, int lane, float (&va)[8], float (&vb)[8]) const
    {
        const int r = r0 + 2 * warp;
        const bool live = r < rend;
        const int tap = live ? r / O8 : 0;
        const int o0 = r - tap * O8;
        const int dh = tap_dh[tap], dw_ = tap_dw[tap], ij = tap_ij[tap];
        const int ohw = g.OH * g.OW;
        float sc[2], zz[2];
        bool o_ok[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            o_ok[e] = live && o0 + e < O;
            sc[e] = (o_ok[e] && gs != nullptr) ? __ldg(gs + o0 + e) : 1.0f;
            zz[e] = (o_ok[e] && wz != nullptr) ? __ldg(wz + o0 + e) : 0.0f;
        }
#pragma unroll
        for (int rg = 0; rg < 4; ++rg) {
            const int th = hp[rg] - dh, tw = wp[rg] - dw_;
            unsigned oh = th, ow = tw;
            if (g.SH != 1) oh = tc_div(th < 0 ? 0 : th, divSH);
            if (g.SW != 1) ow = tc_div(tw < 0 ? 0 : tw, divSW);
            const bool hit = th >= 0 && tw >= 0 && oh < static_cast<unsigned>(g.OH) && ow < static_cast<unsigned>(g.OW);
            const int a_off = go_n[rg] + static_cast<int>(oh) * g.OW + static_cast<int>(ow);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                va[2 * rg + e] = (hit && o_ok[e]) ? __ldg(go + a_off + (o0 + e) * ohw) * sc[e] : 0.0f;
                vb[2 * rg + e] = (o_ok[e] && ckk[rg] >= 0) ? tab[__ldg(widx + (o0 + e) * K + ckk[rg] + ij)] - zz[e] : 0.0f;
            }
        }
    }
    template <bool EXACT_B>
    __device__ void store(uint8_t* stage, const float (&va)[8], const float (&vb)[8]) const
    {
#pragma unroll
        for (int rg = 0; rg < 4; ++rg) {
            uint32_t hi, mid, lo;
            tc_split2(va[2 * rg], va[2 * rg + 1], hi, mid, lo);
            *reinterpret_cast<uint32_t*>(stage + soff[rg]) = hi;
            *reinterpret_cast<uint32_t*>(stage + TcSplitBytes + soff[rg]) = mid;
            *reinterpret_cast<uint32_t*>(stage + 2 * TcSplitBytes + soff[rg]) = lo;
            if (EXACT_B) {
                const __nv_bfloat162 pb = __floats2bfloat162_rn(vb[2 * rg], vb[2 * rg + 1]);
                *reinterpret_cast<uint32_t*>(stage + 3 * TcSplitBytes + soff[rg]) = *reinterpret_cast<const uint32_t*>(&pb);
            } else {
                tc_split2(vb[2 * rg], vb[2 * rg + 1], hi, mid, lo);
                *reinterpret_cast<uint32_t*>(stage + 3 * TcSplitBytes + soff[rg]) = hi;
                *reinterpret_cast<uint32_t*>(stage + 4 * TcSplitBytes + soff[rg]) = mid;
                *reinterpret_cast<uint32_t*>(stage + 5 * TcSplitBytes + soff[rg]) = lo;
            }
        }
    }
    __device__ void finish(int m, int c, float v) const
    {
        int n, h, w;
        pixel_of(m, n, h, w);
        const int at = ((n * g.C + c) * g.H + h) * g.W + w;
        if (xmask != nullptr) v = (xmask[at] ? v : 0.0f) / fmaxf(__ldg(xscale), 1e-12f);
        gx[at] = v;
    }
};

// ---- the kernel -------------------------------------------------------------------------------------------------------------
// EXACT_B: operand B is exactly representable in bf16 (only its hi term is produced and multiplied).
template <class Prob, bool EXACT_B>
__global__ void __launch_bounds__(TcThreads, 2) tc_gemm_kernel(const Prob prob_in)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint32_t s_tmem;
    __shared__ __align__(8) uint64_t s_bar[2];
    Prob p = prob_in;
    int rbeg, rend;
    p.setup(blockIdx.z, gridDim.z, rbeg, rend);
    const int M = p.M(), N = p.N();
    const int m0 = blockIdx.x * TcM, n0 = blockIdx.y * TcN;
    if (m0 >= M) return;                                  // stride classes differ in size: surplus blocks leave
    if (Prob::kAtomic && rbeg >= rend) return;            // nothing to add
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = static_cast<uint32_t>(__cvta_generic_to_shared(&s_bar[0]));
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;"
                     ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s_tmem))) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const uint32_t smem_a = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

    p.prep(warp, lane, m0, n0);
    const int ntiles = (rend - rbeg + TcK - 1) / TcK;
    bool healthy = true;
    // The raw operand values of the NEXT slice are fetched right after this slice's have been stored, so that their
    // global-memory latency runs under the barrier, the MMA issue and the wait for the stage to become free.
    // One slice: wait until the stage is free, store the slice's operand terms, start loading the next slice into
    // the same registers, fence, barrier, and let thread 0 issue the MMAs. (A variant with two slices in flight in
    // two register sets at one block per SM measured 25 % slower: the second resident block hides more latency.)
    float va[8], vb[8];
    if (ntiles > 0) p.load(rbeg, rend, warp, lane, va, vb);
    for (int t = 0; t < ntiles; ++t) {
        const int s = t & 1;
        if (t >= 2 && !tc_wait(bar0 + 8 * s, ((t >> 1) - 1) & 1)) healthy = false;     // the MMAs that read this stage are done
        p.template store<EXACT_B>(smem + s * TcStageBytes, va, vb);
        if (t + 1 < ntiles) p.load(rbeg + (t + 1) * TcK, rend, warp, lane, va, vb);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // generic-proxy writes -> visible to the tensor core
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = smem_a + s * TcStageBytes;
#pragma unroll
            for (int ks = 0; ks < TcK / 16; ++ks) {
                const uint32_t kstep = ks * 2 * TcLBO;
                const uint64_t a_hi = tc_desc(sa + kstep), a_mid = tc_desc(sa + TcSplitBytes + kstep), a_lo = tc_desc(sa + 2 * TcSplitBytes + kstep);
                const uint64_t b_hi = tc_desc(sa + 3 * TcSplitBytes + kstep);
                tc_mma(tmem, a_hi, b_hi, t > 0 || ks > 0);
                tc_mma(tmem, a_mid, b_hi, true);
                tc_mma(tmem, a_lo, b_hi, true);
                if (!EXACT_B) {
                    const uint64_t b_mid = tc_desc(sa + 4 * TcSplitBytes + kstep), b_lo = tc_desc(sa + 5 * TcSplitBytes + kstep);
                    tc_mma(tmem, a_hi, b_mid, true);
                    tc_mma(tmem, a_mid, b_mid, true);
                    tc_mma(tmem, a_hi, b_lo, true);
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar0 + 8 * s) : "memory");
        }
    }
    // every MMA is complete when the last use of each stage has arrived
    for (int s = 0; s < 2; ++s) {
        const int uses = (ntiles + 1 - s) / 2;
        if (uses > 0 && !tc_wait(bar0 + 8 * s, (uses - 1) & 1)) healthy = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!healthy) atomicExch(&g_tc_status, 1);
    if (ntiles > 0 && healthy) {
        // warp w reads TMEM lanes 32 (w % 4) .. + 31 (the tile rows) and columns 32 (w / 4) .. + 31
        const int q = warp & 3, chunk = warp >> 2;
        uint32_t r[32];
        const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(chunk * 32);
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                       "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                       "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                       "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                     : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int m = m0 + q * 32 + lane;
        if (m < M) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int n = n0 + chunk * 32 + j;
                if (n < N) p.finish(m, n, __uint_as_float(r[j]));
            }
        }
    } else if (ntiles == 0 && !Prob::kAtomic) {
        // empty reduction: the tile is zero
        const int q = warp & 3, chunk = warp >> 2;
        const int m = m0 + q * 32 + lane;
        if (m < M)
            for (int j = 0; j < 32; ++j) {
                const int n = n0 + chunk * 32 + j;
                if (n < N) p.finish(m, n, 0.0f);
            }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmem) : "memory");
}

template <class Prob, bool EXACT_B>
static int tc_launch(const Prob& p, long long M, long long N, unsigned gz, cudaStream_t s)
{
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return ATB_ERR_CUDA;
    }
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(tc_gemm_kernel<Prob, EXACT_B>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmemBytes);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        attr_set[dev] = true;
    }
    const dim3 grid(ceil_div(M, TcM), ceil_div(N, TcN), gz);
    if (grid.y > 65535 || grid.z > 65535) return fail_invalid("problem too large for the tensor-core backward");
    tc_gemm_kernel<Prob, EXACT_B><<<grid, TcThreads, TcSmemBytes, s>>>(p);
    return check_launch("tc_gemm_kernel");
}

// Slices of the pixel axis per output tile: as many as keep every block resident at once (two blocks per SM), so
// that no block runs in a second, nearly empty wave.
static int tc_split_factor(long long tiles, long long P)
{
    const long long slots = 2LL * sm_count();
    long long s = tiles >= slots ? 1 : slots / tiles;
    const long long maxs = (P + 8 * TcK - 1) / (8 * TcK);
    if (s > maxs) s = maxs;
    if (s > 1024) s = 1024;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

int tc_conv_grad_w(const float* go, const void* x, int x_dtype, const float* dw, const float* go_scale, float* grad_w,
                   int N, int O, const ConvGeom& g, int pad_index, bool exact_tables, cudaStream_t s)
{
    const int K = g.C * g.KH * g.KW;
    const long long P = static_cast<long long>(N) * g.OH * g.OW;
    const long long tiles = static_cast<long long>(ceil_div(O, TcM)) * ceil_div(K, TcN);
    const unsigned gz = tc_split_factor(tiles, P);
    const TcFastDiv dL = tc_fastdiv(g.OH * g.OW), dOW = tc_fastdiv(g.OW), dKK = tc_fastdiv(g.KH * g.KW), dKW = tc_fastdiv(g.KW);
#define ATB_TC_GW(DT)                                                                                                   \
    {                                                                                                                   \
        TcGradW<DT> p{go, x, dw, go_scale, grad_w, O, K, pad_index, N, P, g, dL, dOW, dKK, dKW};                         \
        return exact_tables ? tc_launch<TcGradW<DT>, true>(p, O, K, gz, s) : tc_launch<TcGradW<DT>, false>(p, O, K, gz, s); \
    }
    if (x_dtype == ATB_U8) ATB_TC_GW(ATB_U8)
    if (x_dtype == ATB_I8) ATB_TC_GW(ATB_I8)
    ATB_TC_GW(ATB_F32)
#undef ATB_TC_GW
}

int tc_conv_grad_x(const float* go, const uint8_t* widx, const float* dx, const float* go_scale, const float* w_zero,
                   const uint8_t* x_mask, const float* x_scale, float* grad_x, int N, int O, const ConvGeom& g,
                   bool exact_tables, cudaStream_t s)
{
    const int K = g.C * g.KH * g.KW;
    TcGradX p{go, widx, dx, go_scale, w_zero, grad_x, N, O, K, (O + 7) / 8 * 8, g, tc_fastdiv(g.SH), tc_fastdiv(g.SW),
              x_mask, x_scale};
    const long long max_class = static_cast<long long>(N) * ((g.H + g.SH - 1) / g.SH) * ((g.W + g.SW - 1) / g.SW);
    return exact_tables ? tc_launch<TcGradX, true>(p, max_class, g.C, g.SH * g.SW, s)
                        : tc_launch<TcGradX, false>(p, max_class, g.C, g.SH * g.SW, s);
}

// =====================================================================================================================
// Second form: operands packed ahead of the contraction, persistent warp-specialised kernel
// =====================================================================================================================
// The kernels above rebuild the three bf16 terms of every gradient value once per tap that reads it and store them two
// bytes at a time: they are bound by the instructions that produce the operands, not by the tensor cores.  When the
// caller provides scratch memory the gradient is instead split ONCE by a streaming pass into bf16 planes laid out the
// way each contraction reads them,
//   GX[term][pixel p = (n, oh, ow)][o]   (o padded to a multiple of 64)     for grad_x: 64 consecutive o = one 128-byte row
//   GW[term][o][p]                       (row pitch a multiple of 8)        for grad_w: 64 consecutive p = one 128-byte row
// and the mapped weights of grad_x into WT[term][tap][c][o].  A 64-element slice of the reduction is then one
// 128-byte row per tile row, which is the K-major layout with 128-byte swizzle that tcgen05.mma reads (8-row atoms of
// 1024 bytes, the 16-byte chunk c of row r stored at chunk c ^ (r & 7)): a warp's asynchronous 16-byte copies
// (cp.async, zero fill outside the image) read whole 128-byte lines and write whole 128-byte shared-memory rows.
// Only grad_w's image operand (the table map of the saved 8-bit activations under the window shift) is still
// produced by the threads, 8 consecutive pixels per item.
//
// One block per SM walks over the output tiles (tile t = blockIdx.x + i * gridDim.x).  Roles by warp:
//   warps 0-3   epilogue: read a finished accumulator out of TMEM (tcgen05.ld) and store / atomically add it;
//   warp  4     one thread issues the MMAs of a slice as soon as its stage is full, and commits to the stage's
//               "empty" barrier (and, after a tile's last slice, to the accumulator's "full" barrier);
//   warps 5-20  producers: wait until a stage is empty, fill it, and - one slice later, when their own copies have
//               landed and are fenced for the asynchronous proxy - arrive on the stage's "full" barrier.
// Two accumulators (2 x 128 TMEM columns) let the epilogue of one tile run under the MMAs of the next; no block-wide
// barrier sits in the loop.  Every wait is bounded: a role that gives up raises a block-wide abort flag (all other
// waits poll it), the status word is set, and the block leaves through the common exit.
// grad_w is computed transposed (rows = (c, tap), columns = o) so that rows fill 128-row tiles whatever O is and the
// atomics of a warp fall on consecutive addresses; N is 64 instead of 128 when the column operand has at most 64 rows.

constexpr int PkK = 64;                              // reduction slice: one 128-byte swizzle row of bf16
constexpr int PkTermBytes = 128 * 128;               // one bf16 term of one 128-row operand tile
constexpr int PkEpiWarps = 4, PkProdWarps = 16;
constexpr int PkThreads = 32 * (PkEpiWarps + 1 + PkProdWarps);     // 672
// producer thread p (0 .. 511) fills chunk p & 7 of rows p >> 3 and (p >> 3) + 64 of every operand tile

__device__ __forceinline__ void tc_mma_n(uint32_t tmem, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate)
{
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// K-major operand with 128-byte swizzle: 8-row atoms 1024 bytes apart (the leading-dimension field is unused)
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t saddr)
{
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
// 16 bytes global -> shared, asynchronously; `bytes` < 16 zero-fills the rest (0: nothing is read)
__device__ __forceinline__ void tc_copy16(uint32_t dst, const void* src, int bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait that also gives up when another role of the block has
__device__ __forceinline__ bool tc_wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (int i = 0; i < (1 << 21); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// ---- the packing pass over the gradient ------------------------------------------------------------------------------------
// One block = 32 channels x 32 pixels of one sample, 256 threads; v = go * gs[o] is split once and written to both
// plane sets.  VEC: L % 4 == 0 and 16-byte aligned go, so that a thread reads four consecutive pixels of a channel at
// once and writes them as one 8-byte piece per term of GW, and - after the turn through shared memory - four
// consecutive channels of a pixel as one 8-byte piece per term of GX.
template <bool VEC>
__global__ void __launch_bounds__(256) tc_pack_go_kernel(const float* __restrict__ go, const float* __restrict__ gs,
                                                         uint16_t* __restrict__ gx_planes, uint16_t* __restrict__ gw_planes,
                                                         int O, int L, int Opad, long long P, long long Ppad)
{
    __shared__ __align__(8) uint16_t tile[3][32][36];               // [term][pixel][channel], 8-byte aligned rows
    const int l0 = blockIdx.x * 32, o0 = blockIdx.y * 32, n = blockIdx.z;
    const int t = threadIdx.x;
    const long long gx_plane = P * Opad, gw_plane = static_cast<long long>(O) * Ppad;
    {
        const int o = o0 + (t >> 3), l = l0 + 4 * (t & 7);
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (o < O) {
            const float* src = go + (static_cast<long long>(n) * O + o) * L + l;
            if (VEC) {
                if (l < L) { const float4 f = __ldcs(reinterpret_cast<const float4*>(src)); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) if (l + e < L) v[e] = __ldcs(src + e);
            }
            if (gs != nullptr) { const float sc = __ldg(gs + o); v[0] *= sc; v[1] *= sc; v[2] *= sc; v[3] *= sc; }
        }
        uint32_t h01, m01, l01, h23, m23, l23;
        tc_split2(v[0], v[1], h01, m01, l01);
        tc_split2(v[2], v[3], h23, m23, l23);
        if (gw_planes != nullptr && o < O && l < L) {
            const long long at = o * Ppad + static_cast<long long>(n) * L + l;
            if (VEC) {
                *reinterpret_cast<uint2*>(gw_planes + at) = make_uint2(h01, h23);
                *reinterpret_cast<uint2*>(gw_planes + gw_plane + at) = make_uint2(m01, m23);
                *reinterpret_cast<uint2*>(gw_planes + 2 * gw_plane + at) = make_uint2(l01, l23);
            } else {
                const uint32_t hh[2] = {h01, h23}, mm[2] = {m01, m23}, ll[2] = {l01, l23};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (l + e < L) {
                        gw_planes[at + e] = static_cast<uint16_t>(hh[e >> 1] >> (16 * (e & 1)));
                        gw_planes[gw_plane + at + e] = static_cast<uint16_t>(mm[e >> 1] >> (16 * (e & 1)));
                        gw_planes[2 * gw_plane + at + e] = static_cast<uint16_t>(ll[e >> 1] >> (16 * (e & 1)));
                    }
            }
        }
        const int oc = t >> 3, lp = 4 * (t & 7);
        tile[0][lp][oc] = static_cast<uint16_t>(h01); tile[0][lp + 1][oc] = static_cast<uint16_t>(h01 >> 16);
        tile[0][lp + 2][oc] = static_cast<uint16_t>(h23); tile[0][lp + 3][oc] = static_cast<uint16_t>(h23 >> 16);
        tile[1][lp][oc] = static_cast<uint16_t>(m01); tile[1][lp + 1][oc] = static_cast<uint16_t>(m01 >> 16);
        tile[1][lp + 2][oc] = static_cast<uint16_t>(m23); tile[1][lp + 3][oc] = static_cast<uint16_t>(m23 >> 16);
        tile[2][lp][oc] = static_cast<uint16_t>(l01); tile[2][lp + 1][oc] = static_cast<uint16_t>(l01 >> 16);
        tile[2][lp + 2][oc] = static_cast<uint16_t>(l23); tile[2][lp + 3][oc] = static_cast<uint16_t>(l23 >> 16);
    }
    if (gx_planes == nullptr) return;
    __syncthreads();
    {
        const int l = l0 + (t >> 3), oq = 4 * (t & 7);              // four consecutive channels of one pixel: 8 bytes per term
        if (l < L) {
            const long long at = (static_cast<long long>(n) * L + l) * Opad + o0 + oq;
#pragma unroll
            for (int term = 0; term < 3; ++term)
                *reinterpret_cast<uint2*>(gx_planes + term * gx_plane + at) = *reinterpret_cast<const uint2*>(&tile[term][t >> 3][oq]);
        }
    }
}

// WT[term][tap][c][o] = split(dx[widx[o, c, tap]] - wz[o]); zero for o >= O.  One thread per (tap, c, o).
__global__ void tc_pack_w_kernel(const uint8_t* __restrict__ widx, const float* __restrict__ dx, const float* __restrict__ wz,
                                 uint16_t* __restrict__ wt, int O, int C, int KK, int Opad, int terms)
{
    const long long total = static_cast<long long>(KK) * C * Opad;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int o = static_cast<int>(i % Opad);
        const long long tc = i / Opad;
        const int c = static_cast<int>(tc % C), tap = static_cast<int>(tc / C);
        uint16_t hi = 0, mid = 0, lo = 0;
        if (o < O) {
            float v = __ldg(dx + __ldg(widx + (static_cast<long long>(o) * C + c) * KK + tap));
            if (wz != nullptr) v -= __ldg(wz + o);
            tc_split1(v, hi, mid, lo);
        }
        wt[i] = hi;
        if (terms == 3) { wt[total + i] = mid; wt[2 * total + i] = lo; }
    }
}

// ---- problem: grad_x from packed planes ----------------------------------------------------------------------------------
// rows: the pixels of one stride class z; columns: c; reduction index r = tap * Opad + o over the class's taps.
struct PkGradX {
    const uint16_t* gxp; const uint16_t* wt; float* gx;
    int Nb, Opad, classes; ConvGeom g;
    TcFastDiv divSH, divSW;
    const uint8_t* xmask; const float* xscale;
    long long gx_plane, wt_plane;
    int mt, nt;                                  // tiles along the rows (of the largest class) and along c
    static constexpr bool kAtomic = false;
    // block state (shared memory): the taps of every class
    const int* cls_start; const int* tap_dh; const int* tap_dw; const int* tap_ij;
    __device__ void block_setup()
    {
        __shared__ int s_start[65], s_dh[TcMaxTaps], s_dw[TcMaxTaps], s_ij[TcMaxTaps];
        if (threadIdx.x == 0) {
            int n = 0;
            for (int z = 0; z < classes; ++z) {
                s_start[z] = n;
                const int a = z / g.SW, b = z - a * g.SW;
                for (int i = 0; i < g.KH; ++i) {
                    if (((a - i * g.DH) % g.SH + g.SH) % g.SH != 0) continue;
                    for (int j = 0; j < g.KW; ++j) {
                        if (((b - j * g.DW) % g.SW + g.SW) % g.SW != 0) continue;
                        s_dh[n] = i * g.DH; s_dw[n] = j * g.DW; s_ij[n] = i * g.KW + j; ++n;
                    }
                }
            }
            s_start[classes] = n;
        }
        cls_start = s_start; tap_dh = s_dh; tap_dw = s_dw; tap_ij = s_ij;
    }
    __device__ long long tiles() const { return static_cast<long long>(mt) * nt * classes; }
    struct Tile { int m0, n0, z, rbeg, rend, M, h0, w0, Hc, Wc; };
    __device__ Tile tile(long long t, int ncols) const
    {
        Tile T;
        const int per = mt * nt;
        T.z = static_cast<int>(t / per);
        const int rem = static_cast<int>(t - static_cast<long long>(T.z) * per);
        const int ni = rem / mt;
        T.m0 = (rem - ni * mt) * TcM; T.n0 = ni * ncols;
        const int a = T.z / g.SW, b = T.z - a * g.SW;
        T.h0 = ((a - g.PH) % g.SH + g.SH) % g.SH;
        T.w0 = ((b - g.PW) % g.SW + g.SW) % g.SW;
        T.Hc = T.h0 < g.H ? (g.H - T.h0 + g.SH - 1) / g.SH : 0;
        T.Wc = T.w0 < g.W ? (g.W - T.w0 + g.SW - 1) / g.SW : 0;
        T.M = Nb * T.Hc * T.Wc;
        T.rbeg = 0; T.rend = (cls_start[T.z + 1] - cls_start[T.z]) * Opad;
        return T;
    }
    __device__ int N() const { return g.C; }
    __device__ void pixel_of(const Tile& T, int m, int& n, int& h, int& w) const
    {
        const int hw = T.Hc * T.Wc;
        n = m / hw;
        const int rem = m - n * hw;
        const int t = rem / T.Wc;
        h = T.h0 + g.SH * t;
        w = T.w0 + g.SW * (rem - t * T.Wc);
    }
    // per-thread producer state of a tile: two rows (row0, row0 + 64)
    struct Rows { int hp[2], wp[2]; long long pix_base[2]; int c_row[2]; };
    __device__ Rows rows(const Tile& T, int p) const
    {
        Rows R;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = (p >> 3) + 64 * i;
            const int m = T.m0 + row;
            R.hp[i] = R.wp[i] = -(1 << 28);
            R.pix_base[i] = 0;
            if (m < T.M) {
                int n, h, w;
                pixel_of(T, m, n, h, w);
                R.hp[i] = h + g.PH; R.wp[i] = w + g.PW;
                R.pix_base[i] = static_cast<long long>(n) * g.OH * g.OW;
            }
            R.c_row[i] = T.n0 + row < g.C ? T.n0 + row : -1;
        }
        return R;
    }
    template <int NA, int NB>
    __device__ void produce(uint32_t stage, const Tile& T, const Rows& R, int r0, int p, int ncols) const
    {
        const int tap_l = r0 / Opad;
        const int tap = cls_start[T.z] + tap_l;
        const int o0 = r0 - tap_l * Opad + 8 * (p & 7);
        const int dh = tap_dh[tap], dw_ = tap_dw[tap];
        const long long b_tap = static_cast<long long>(tap_ij[tap]) * g.C;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = (p >> 3) + 64 * i;
            const uint32_t dst = stage + static_cast<uint32_t>(row) * 128u + static_cast<uint32_t>(((p & 7) ^ (row & 7)) << 4);
            const int th = R.hp[i] - dh, tw = R.wp[i] - dw_;
            unsigned oh = th, ow = tw;
            if (g.SH != 1) oh = tc_div(th < 0 ? 0 : th, divSH);
            if (g.SW != 1) ow = tc_div(tw < 0 ? 0 : tw, divSW);
            const bool hit = th >= 0 && tw >= 0 && oh < static_cast<unsigned>(g.OH) && ow < static_cast<unsigned>(g.OW);
            const uint16_t* a = gxp + (hit ? (R.pix_base[i] + oh * g.OW + ow) * Opad + o0 : 0LL);
#pragma unroll
            for (int t = 0; t < NA; ++t) tc_copy16(dst + t * PkTermBytes, a + t * gx_plane, hit ? 16 : 0);
            if (row < ncols) {
                const bool ok = R.c_row[i] >= 0;
                const uint16_t* b = wt + (ok ? (b_tap + R.c_row[i]) * Opad + o0 : 0LL);
#pragma unroll
                for (int t = 0; t < NB; ++t) tc_copy16(dst + (NA + t) * PkTermBytes, b + t * wt_plane, ok ? 16 : 0);
            }
        }
    }
    // epilogue state of a thread (its row) and the store of one element
    struct Out { int base; bool ok; };
    __device__ Out out_row(const Tile& T, int m) const
    {
        Out o{0, m < T.M};
        if (o.ok) {
            int n, h, w;
            pixel_of(T, m, n, h, w);
            o.base = (n * g.C * g.H + h) * g.W + w;
        }
        return o;
    }
    __device__ void finish(const Out& o, int c, float v) const
    {
        const int at = o.base + c * g.H * g.W;
        if (xmask != nullptr) v = (xmask[at] ? v : 0.0f) / fmaxf(__ldg(xscale), 1e-12f);
        gx[at] = v;
    }
};

// ---- problem: grad_w (transposed) from the packed gradient -------------------------------------------------------------------
// rows: k = (c, tap), produced by the threads from the saved 8-bit image through the table; columns: o, copied from
// GW; reduction over the pixels of slice z of the pixel axis.  Result element (k, o) is added to grad_w[o, k].
template <int XDT>
struct PkGradW {
    const void* x; const float* dw; const uint16_t* gwp; float* gw; float* part;
    int O, K, pad_index, gz; long long P, Ppad, gw_plane; ConvGeom g;
    TcFastDiv divL, divOW, divKK, divKW, divKH;
    int mt, nt, window;
    static constexpr bool kAtomic = true;
    const uint16_t* t_hi; const uint16_t* t_mid; const uint16_t* t_lo;      // the table's bf16 terms in shared memory
    __device__ void block_setup()
    {
        __shared__ uint16_t s_hi[257], s_mid[257], s_lo[257];
        for (int i = threadIdx.x; i < 257; i += blockDim.x) {
            uint16_t hi, mid, lo;
            tc_split1(__ldg(dw + (i < 256 || pad_index == 256 ? i : 255)), hi, mid, lo);
            s_hi[i] = hi; s_mid[i] = mid; s_lo[i] = lo;
        }
        t_hi = s_hi; t_mid = s_mid; t_lo = s_lo;
    }
    __device__ long long tiles() const { return static_cast<long long>(mt) * nt * gz; }
    struct Tile { int m0, n0, z, rbeg, rend, M; };
    __device__ Tile tile(long long t, int ncols) const
    {
        Tile T;
        const int per = mt * nt;
        T.z = static_cast<int>(t / per);
        const int rem = static_cast<int>(t - static_cast<long long>(T.z) * per);
        const int ni = rem / mt;
        T.m0 = (rem - ni * mt) * TcM; T.n0 = ni * ncols;
        T.M = K;
        const long long per_z = ((P + gz - 1) / gz + PkK - 1) / PkK * PkK;
        const long long b0 = per_z * T.z;
        T.rbeg = static_cast<int>(b0 < P ? b0 : P);
        T.rend = static_cast<int>(b0 + per_z < P ? b0 + per_z : P);
        return T;
    }
    __device__ int N() const { return O; }
    // per-thread producer state of a tile.  Generic mapping: two rows (row0, row0 + 64), one 8-pixel chunk each.
    // Window mapping (stride and dilation 1 along w, 2 or 3 taps per kernel row): thread p owns the KW rows of
    // group (c, i) number p >> 3 of the tile and one chunk - the taps of a kernel row read the same stretch of the
    // image shifted by one, so 8 + KW - 1 table lookups feed 8 * KW elements.
    struct Rows { int k_c[2], k_dh[2], k_dw[2], o_row[2]; int w_c, w_dh, w_row0; };
    __device__ Rows rows(const Tile& T, int p) const
    {
        Rows R;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = (p >> 3) + 64 * i;
            const int k = T.m0 + row;
            R.k_c[i] = -1; R.k_dh[i] = R.k_dw[i] = 0;
            if (k < K) {
                const unsigned c = tc_div(k, divKK);
                const unsigned ij = k - c * (g.KH * g.KW);
                const unsigned ti = tc_div(ij, divKW);
                R.k_c[i] = static_cast<int>(c);
                R.k_dh[i] = static_cast<int>(ti) * g.DH - g.PH;
                R.k_dw[i] = static_cast<int>(ij - ti * g.KW) * g.DW - g.PW;
            }
            R.o_row[i] = T.n0 + row < O ? T.n0 + row : -1;
        }
        R.w_c = -1; R.w_dh = 0; R.w_row0 = 0;
        if (window) {
            const int grp = static_cast<int>(tc_div(T.m0, divKW)) + (p >> 3);          // (c, i) pair number
            const int k0 = grp * g.KW;
            if (k0 < T.m0 + TcM && k0 < K) {
                const unsigned c = tc_div(grp, divKH);
                R.w_c = static_cast<int>(c);
                R.w_dh = (grp - static_cast<int>(c) * g.KH) * g.DH - g.PH;
                R.w_row0 = k0 - T.m0;                                                   // may be negative: rows of the tile before
            }
        }
        return R;
    }
    // eight consecutive pixels of tap (kdh, kdw) of channel kc through the table, into chunk `dst` of the row's terms
    template <int NA>
    __device__ void row_generic(uint32_t dst, int kc, int kdh, int kdw, unsigned n, int oh, int ow, int left) const
    {
        uint32_t hi[4] = {0u, 0u, 0u, 0u}, mid[4] = {0u, 0u, 0u, 0u}, lo[4] = {0u, 0u, 0u, 0u};
        if (kc >= 0 && left > 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (e < left) {
                    const int ih = oh * g.SH + kdh, iw = ow * g.SW + kdw;
                    int idx = pad_index;
                    if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
                        idx = index_of<XDT>(x, ((static_cast<int>(n) * g.C + kc) * g.H + ih) * g.W + iw);
                    hi[e >> 1] |= static_cast<uint32_t>(t_hi[idx]) << (16 * (e & 1));
                    if (NA == 3) {
                        mid[e >> 1] |= static_cast<uint32_t>(t_mid[idx]) << (16 * (e & 1));
                        lo[e >> 1] |= static_cast<uint32_t>(t_lo[idx]) << (16 * (e & 1));
                    }
                }
                if (++ow == g.OW) { ow = 0; if (++oh == g.OH) { oh = 0; ++n; } }
            }
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
        if (NA == 3) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + PkTermBytes), "r"(mid[0]), "r"(mid[1]), "r"(mid[2]), "r"(mid[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 2 * PkTermBytes), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
        }
    }
    template <int NA, int NB>
    __device__ void produce(uint32_t stage, const Tile& T, const Rows& R, int r0, int p, int ncols) const
    {
        const int chunk = p & 7;
        const int p0 = r0 + 8 * chunk;
        const int left = T.rend - p0;
        // where the chunk's first pixel lies
        const int L = g.OH * g.OW;
        const int pc = left > 0 ? p0 : 0;
        const unsigned n0 = tc_div(pc, divL);
        const int l0 = pc - static_cast<int>(n0) * L;
        const int oh0 = static_cast<int>(tc_div(l0, divOW));
        const int ow0 = l0 - oh0 * g.OW;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = (p >> 3) + 64 * i;
            const uint32_t dst = stage + static_cast<uint32_t>(row) * 128u + static_cast<uint32_t>((chunk ^ (row & 7)) << 4);
            // columns: 16 bytes of each plane of GW (clipped at the end of this tile's share of the pixels)
            if (row < ncols) {
                const int bytes = (R.o_row[i] >= 0 && left > 0) ? (left >= 8 ? 16 : 2 * left) : 0;
                const uint16_t* b = gwp + (bytes > 0 ? R.o_row[i] * Ppad + p0 : 0LL);
#pragma unroll
                for (int t = 0; t < NB; ++t) tc_copy16(dst + (NA + t) * PkTermBytes, b + t * gw_plane, bytes);
            }
            if (!window) row_generic<NA>(dst, R.k_c[i], R.k_dh[i], R.k_dw[i], n0, oh0, ow0, left);
        }
        if (!window || R.w_c < 0) return;
        const int kw = g.KW;
        if (left >= 8 && ow0 + 8 <= g.OW) {
            // one stretch of 8 + kw - 1 image bytes serves the kw taps of the kernel row
            const int ih = oh0 * g.SH + R.w_dh;
            const bool row_ok = static_cast<unsigned>(ih) < static_cast<unsigned>(g.H);
            const int base = ((static_cast<int>(n0) * g.C + R.w_c) * g.H + (row_ok ? ih : 0)) * g.W;
            const int iw0 = ow0 - g.PW;
            uint32_t vh[10], vm[10], vl[10];
#pragma unroll
            for (int q = 0; q < 10; ++q) {
                vh[q] = vm[q] = vl[q] = 0u;
                if (q < 8 + kw - 1) {
                    const int iw = iw0 + q;
                    int idx = pad_index;
                    if (row_ok && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W)) idx = index_of<XDT>(x, base + iw);
                    vh[q] = t_hi[idx];
                    if (NA == 3) { vm[q] = t_mid[idx]; vl[q] = t_lo[idx]; }
                }
            }
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int row = R.w_row0 + j;
                if (j < kw && row >= 0 && row < TcM) {
                    const uint32_t dst = stage + static_cast<uint32_t>(row) * 128u + static_cast<uint32_t>((chunk ^ (row & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(vh[j] | (vh[j + 1] << 16)), "r"(vh[j + 2] | (vh[j + 3] << 16)),
                                 "r"(vh[j + 4] | (vh[j + 5] << 16)), "r"(vh[j + 6] | (vh[j + 7] << 16)) : "memory");
                    if (NA == 3) {
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + PkTermBytes), "r"(vm[j] | (vm[j + 1] << 16)),
                                     "r"(vm[j + 2] | (vm[j + 3] << 16)), "r"(vm[j + 4] | (vm[j + 5] << 16)), "r"(vm[j + 6] | (vm[j + 7] << 16)) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 2 * PkTermBytes), "r"(vl[j] | (vl[j + 1] << 16)),
                                     "r"(vl[j + 2] | (vl[j + 3] << 16)), "r"(vl[j + 4] | (vl[j + 5] << 16)), "r"(vl[j + 6] | (vl[j + 7] << 16)) : "memory");
                    }
                }
            }
        } else {
            // a chunk that crosses the end of an image row (or of this tile's share): pixel by pixel with a sliding
            // window over the kernel row's taps - one new lookup per pixel, kw at the start of an image row
            uint32_t th[3][4] = {}, tm[3][4] = {}, tl[3][4] = {};
            uint32_t wh[3] = {0u, 0u, 0u}, wm[3] = {0u, 0u, 0u}, wl[3] = {0u, 0u, 0u};
            unsigned n = n0;
            int oh = oh0, ow = ow0, base = 0;
            bool fresh = true, row_ok = false;
            auto look = [&](int iw, int slot) {
                int idx = pad_index;
                if (row_ok && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W)) idx = index_of<XDT>(x, base + iw);
                wh[slot] = t_hi[idx];
                if (NA == 3) { wm[slot] = t_mid[idx]; wl[slot] = t_lo[idx]; }
            };
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (e < left) {
                    if (fresh) {
                        const int ih = oh * g.SH + R.w_dh;
                        row_ok = static_cast<unsigned>(ih) < static_cast<unsigned>(g.H);
                        base = ((static_cast<int>(n) * g.C + R.w_c) * g.H + (row_ok ? ih : 0)) * g.W;
                        look(ow - g.PW, 0);
                        if (kw == 3) look(ow - g.PW + 1, 1);
                    }
                    if (kw == 3) look(ow - g.PW + 2, 2); else look(ow - g.PW + 1, 1);
#pragma unroll
                    for (int j = 0; j < 3; ++j)
                        if (j < kw) {
                            th[j][e >> 1] |= wh[j] << (16 * (e & 1));
                            if (NA == 3) { tm[j][e >> 1] |= wm[j] << (16 * (e & 1)); tl[j][e >> 1] |= wl[j] << (16 * (e & 1)); }
                        }
                    wh[0] = wh[1]; wm[0] = wm[1]; wl[0] = wl[1];
                    if (kw == 3) { wh[1] = wh[2]; wm[1] = wm[2]; wl[1] = wl[2]; }
                }
                fresh = false;
                if (++ow == g.OW) { ow = 0; fresh = true; if (++oh == g.OH) { oh = 0; ++n; } }
            }
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int row = R.w_row0 + j;
                if (j < kw && row >= 0 && row < TcM) {
                    const uint32_t dst = stage + static_cast<uint32_t>(row) * 128u + static_cast<uint32_t>((chunk ^ (row & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(th[j][0]), "r"(th[j][1]), "r"(th[j][2]), "r"(th[j][3]) : "memory");
                    if (NA == 3) {
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + PkTermBytes), "r"(tm[j][0]), "r"(tm[j][1]), "r"(tm[j][2]), "r"(tm[j][3]) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 2 * PkTermBytes), "r"(tl[j][0]), "r"(tl[j][1]), "r"(tl[j][2]), "r"(tl[j][3]) : "memory");
                    }
                }
            }
        }
    }
    // `part` null: fp32 atomics into the zeroed grad_w (the order of the slices' contributions varies from run to
    // run); otherwise slice z stores its tile into part[z][o][k] and a second pass adds the slices in ascending order
    struct Out { int k; bool ok; int z; };
    __device__ Out out_row(const Tile& T, int m) const { return Out{m, m < K, T.z}; }
    __device__ void finish(const Out& o, int col, float v) const
    {
        if (part != nullptr) part[(static_cast<long long>(o.z) * O + col) * K + o.k] = v;
        else atomicAdd(gw + col * K + o.k, v);
    }
};

// grad_w[i] = sum over the slices z < nz of part[z][i], in ascending z
__global__ void tc_sum_slices_kernel(const float* __restrict__ part, float* __restrict__ gw, int nz, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float acc = 0.0f;
        for (int z = 0; z < nz; ++z) acc += __ldcs(part + z * n + i);
        gw[i] = acc;
    }
}

// NA, NB: bf16 terms of the row and of the column operand (3: hi + mid + lo of an fp32 value, 1: exact in bf16);
// the products (i, j) with i + j <= 2 are issued - lo * mid and smaller fall below fp32 rounding.
template <class Prob, int NA, int NB, int STAGES>
__global__ void __launch_bounds__(PkThreads, 1) tc_packed_kernel(const Prob prob_in, const int ncols)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ __align__(8) uint64_t s_full[STAGES], s_empty[STAGES], s_acc_full[2], s_acc_empty[2];
    constexpr int kStage = (NA + NB) * PkTermBytes;
    Prob p = prob_in;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    p.block_setup();
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s_full[s]))), "r"(PkProdWarps) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s_empty[s]))) : "memory");
        }
        for (int a = 0; a < 2; ++a) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s_acc_full[a]))) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s_acc_empty[a]))), "r"(PkEpiWarps) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;"
                     ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s_tmem))) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // the dynamic area starts on a 1024-byte boundary of the shared window (the swizzle atoms are address based)
    const uint32_t smem_a = (static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw)) + 1023u) & ~1023u;
    const uint32_t full0 = static_cast<uint32_t>(__cvta_generic_to_shared(&s_full[0]));
    const uint32_t empty0 = static_cast<uint32_t>(__cvta_generic_to_shared(&s_empty[0]));
    const uint32_t accf0 = static_cast<uint32_t>(__cvta_generic_to_shared(&s_acc_full[0]));
    const uint32_t acce0 = static_cast<uint32_t>(__cvta_generic_to_shared(&s_acc_empty[0]));
    volatile int* abort_flag = &s_abort;
    const long long ntiles = p.tiles();

    if (warp >= PkEpiWarps + 1) {
        // ---------------------------------------------------------------- producers
        const int pid = tid - 32 * (PkEpiWarps + 1);
        int stage = 0; uint32_t phase = 0;
        int pend_stage[STAGES]; int npend = 0;                   // stages filled by this thread and not yet announced
        bool ok = true;
        for (long long t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
            const typename Prob::Tile T = p.tile(t, ncols);
            if (T.m0 >= T.M || (Prob::kAtomic && T.rbeg >= T.rend)) continue;
            const typename Prob::Rows R = p.rows(T, pid);
            for (int r0 = T.rbeg; r0 < T.rend; r0 += PkK) {
                if (!tc_wait_or_abort(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
                p.template produce<NA, NB>(smem_a + stage * kStage, T, R, r0, pid, ncols);
                asm volatile("cp.async.commit_group;" ::: "memory");
                pend_stage[npend++] = stage;
                if (npend == STAGES - 1) {
                    // the oldest slice: its copies have landed once at most STAGES - 2 newer groups are pending
                    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tc_arrive(full0 + 8 * pend_stage[0]);
#pragma unroll
                    for (int i = 0; i + 1 < STAGES - 1; ++i) pend_stage[i] = pend_stage[i + 1];
                    --npend;
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        for (int i = 0; i < npend; ++i)
            if (lane == 0) tc_arrive(full0 + 8 * pend_stage[i]);
    } else if (warp == PkEpiWarps) {
        // ---------------------------------------------------------------- MMA issue (one thread)
        if (lane == 0) {
            // D fp32, A and B bf16, both K-major, M = 128, N = ncols
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(ncols) >> 3) << 17) | ((128u >> 4) << 24);
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                const typename Prob::Tile T = p.tile(t, ncols);
                if (T.m0 >= T.M || (Prob::kAtomic && T.rbeg >= T.rend)) continue;
                if (T.rbeg < T.rend) {
                    if (!tc_wait_or_abort(acce0 + 8 * acc, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t d = tmem + static_cast<uint32_t>(acc * 128);
                    bool first = true;
                    for (int r0 = T.rbeg; r0 < T.rend; r0 += PkK) {
                        if (!tc_wait_or_abort(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t sa = smem_a + stage * kStage;
#pragma unroll
                        for (int ks = 0; ks < PkK / 16; ++ks) {
#pragma unroll
                            for (int i = 0; i < NA; ++i)
#pragma unroll
                                for (int j = 0; j < NB; ++j)
                                    if (i + j <= 2) {
                                        tc_mma_n(d, tc_desc_sw128(sa + i * PkTermBytes + ks * 32), tc_desc_sw128(sa + (NA + j) * PkTermBytes + ks * 32),
                                                 idesc, !first);
                                        first = false;
                                    }
                        }
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                                     ::"r"(empty0 + 8 * stage) : "memory");
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                                 ::"r"(accf0 + 8 * acc) : "memory");
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warp w: TMEM lanes 32 w .. 32 w + 31)
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
            const typename Prob::Tile T = p.tile(t, ncols);
            if (T.m0 >= T.M || (Prob::kAtomic && T.rbeg >= T.rend)) continue;
            const typename Prob::Out out = p.out_row(T, T.m0 + warp * 32 + lane);
            const int N = p.N();
            if (T.rbeg >= T.rend) {
                // empty reduction: the tile is zero
                if (out.ok)
                    for (int j = 0; j < ncols; ++j)
                        if (T.n0 + j < N) p.finish(out, T.n0 + j, 0.0f);
                continue;
            }
            if (!tc_wait_or_abort(accf0 + 8 * acc, acc_phase, abort_flag)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int c0 = 0; c0 < ncols; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(acc * 128 + c0);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (out.ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = T.n0 + c0 + j;
                        if (n < N) p.finish(out, n, __uint_as_float(r[j]));
                    }
                }
            }
            // this warp is done with the accumulator
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_arrive(acce0 + 8 * acc);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }
    // common exit: nothing of this block is in flight any more (every MMA was committed to a barrier somebody waited
    // on, unless the block aborted), the TMEM columns go back
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && s_abort) atomicExch(&g_tc_status, 1);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
}

template <class Prob, int NA, int NB, int STAGES>
static int tc_packed_launch(const Prob& p, long long tiles, int ncols, cudaStream_t s)
{
    constexpr int kBytes = (NA + NB) * STAGES * PkTermBytes + 1024;       // + room to round the start up to 1024
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return ATB_ERR_CUDA;
    }
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(tc_packed_kernel<Prob, NA, NB, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        attr_set[dev] = true;
    }
    const long long sms = sm_count();
    const int grid = static_cast<int>(tiles < sms ? tiles : sms);
    if (grid <= 0) return ATB_OK;
    tc_packed_kernel<Prob, NA, NB, STAGES><<<grid, PkThreads, kBytes, s>>>(p, ncols);
    return check_launch("tc_packed_kernel");
}

static size_t tc_round256(size_t b) { return (b + 255u) / 256u * 256u; }

// Scratch layout: GX planes | GW planes | WT planes, each 256-byte aligned.
struct TcPackedSizes {
    int Opad; long long P, Ppad; size_t gx_bytes, gw_bytes, wt_bytes, part_bytes;
    int gz, gz_used;           // slices of grad_w's pixel axis, and how many of them are not empty
};
// slices of the pixel axis for grad_w: about two tiles per SM, none shorter than eight 64-pixel steps
static void tc_grad_w_slices(long long K, int O, long long P, int* gz_out, int* used_out)
{
    const int ncols = O <= 64 ? 64 : 128;
    const long long tiles_mn = static_cast<long long>(ceil_div(K, TcM)) * ceil_div(O, ncols);
    long long gz = (2LL * sm_count() + tiles_mn - 1) / tiles_mn;
    const long long maxs = (P + 8 * PkK - 1) / (8 * PkK);
    if (gz > maxs) gz = maxs;
    if (gz > 4096) gz = 4096;
    if (gz < 1) gz = 1;
    const long long per_z = ((P + gz - 1) / gz + PkK - 1) / PkK * PkK;       // as PkGradW::tile cuts the axis
    *gz_out = static_cast<int>(gz);
    *used_out = static_cast<int>(per_z > 0 ? (P + per_z - 1) / per_z : 0);
}
static TcPackedSizes tc_packed_sizes(int N, int O, const ConvGeom& g, bool need_x, bool need_w, bool exact_tables,
                                     bool deterministic)
{
    TcPackedSizes z{};
    z.Opad = (O + PkK - 1) / PkK * PkK;
    z.P = static_cast<long long>(N) * g.OH * g.OW;
    z.Ppad = (z.P + 7) / 8 * 8;
    z.gx_bytes = need_x ? tc_round256(static_cast<size_t>(3) * z.P * z.Opad * 2u) : 0u;
    z.gw_bytes = need_w ? tc_round256(static_cast<size_t>(3) * O * z.Ppad * 2u) : 0u;
    z.wt_bytes = need_x ? tc_round256(static_cast<size_t>(exact_tables ? 1 : 3) * g.KH * g.KW * g.C * z.Opad * 2u) : 0u;
    const long long K = static_cast<long long>(g.C) * g.KH * g.KW;
    tc_grad_w_slices(K, O, z.P, &z.gz, &z.gz_used);
    z.part_bytes = (need_w && deterministic) ? tc_round256(static_cast<size_t>(z.gz_used) * O * K * 4u) : 0u;
    return z;
}

size_t tc_packed_scratch_bytes(int N, int O, const ConvGeom& g, bool need_x, bool need_w, bool exact_tables, bool deterministic)
{
    const TcPackedSizes z = tc_packed_sizes(N, O, g, need_x, need_w, exact_tables, deterministic);
    // 32-bit element offsets inside a plane: larger problems stay on the kernels that build their operands in place
    if (z.P * z.Opad >= 2147483647LL || static_cast<long long>(O) * z.Ppad >= 2147483647LL) return 0;
    return z.gx_bytes + z.gw_bytes + z.wt_bytes + z.part_bytes;
}

// Both gradients (either may be null) from one packing pass.  grad_w must have been zeroed by the caller.
int tc_packed_conv_bwd(const float* go, const void* x, int x_dtype, const uint8_t* widx, const float* dx, const float* dw,
                       const float* go_scale, const float* w_zero, const uint8_t* x_mask, const float* x_scale,
                       float* grad_x, float* grad_w, int N, int O, const ConvGeom& g, int pad_index, bool exact_tables,
                       bool deterministic, void* scratch, cudaStream_t s)
{
    const bool need_x = grad_x != nullptr, need_w = grad_w != nullptr;
    const TcPackedSizes z = tc_packed_sizes(N, O, g, need_x, need_w, exact_tables, deterministic);
    const int L = g.OH * g.OW, KK = g.KH * g.KW, K = g.C * KK;
    uint16_t* gxp = need_x ? static_cast<uint16_t*>(scratch) : nullptr;
    uint16_t* gwp = need_w ? reinterpret_cast<uint16_t*>(static_cast<char*>(scratch) + z.gx_bytes) : nullptr;
    uint16_t* wt = need_x ? reinterpret_cast<uint16_t*>(static_cast<char*>(scratch) + z.gx_bytes + z.gw_bytes) : nullptr;
    float* part = z.part_bytes ? reinterpret_cast<float*>(static_cast<char*>(scratch) + z.gx_bytes + z.gw_bytes + z.wt_bytes) : nullptr;
    {
        const dim3 grid(ceil_div(L, 32), z.Opad / 32, N);
        if (grid.y > 65535 || grid.z > 65535) return fail_invalid("problem too large for the tensor-core backward");
        if (L % 4 == 0 && aligned_to(go, 16)) tc_pack_go_kernel<true><<<grid, 256, 0, s>>>(go, go_scale, gxp, gwp, O, L, z.Opad, z.P, z.Ppad);
        else tc_pack_go_kernel<false><<<grid, 256, 0, s>>>(go, go_scale, gxp, gwp, O, L, z.Opad, z.P, z.Ppad);
        int rc = check_launch("tc_pack_go_kernel");
        if (rc != ATB_OK) return rc;
    }
    if (need_x) {
        const int terms = exact_tables ? 1 : 3;
        const long long total = static_cast<long long>(KK) * g.C * z.Opad;
        tc_pack_w_kernel<<<grid_for(total, 256, 4096), 256, 0, s>>>(widx, dx, w_zero, wt, O, g.C, KK, z.Opad, terms);
        int rc = check_launch("tc_pack_w_kernel");
        if (rc != ATB_OK) return rc;
        const int ncols = g.C <= 64 ? 64 : 128;
        PkGradX p{};
        p.gxp = gxp; p.wt = wt; p.gx = grad_x; p.Nb = N; p.Opad = z.Opad; p.classes = g.SH * g.SW; p.g = g;
        p.divSH = tc_fastdiv(g.SH); p.divSW = tc_fastdiv(g.SW); p.xmask = x_mask; p.xscale = x_scale;
        p.gx_plane = z.P * z.Opad; p.wt_plane = total;
        const long long max_class = static_cast<long long>(N) * ((g.H + g.SH - 1) / g.SH) * ((g.W + g.SW - 1) / g.SW);
        p.mt = ceil_div(max_class, TcM); p.nt = ceil_div(g.C, ncols);
        const long long tiles = static_cast<long long>(p.mt) * p.nt * p.classes;
        rc = exact_tables ? tc_packed_launch<PkGradX, 3, 1, 3>(p, tiles, ncols, s) : tc_packed_launch<PkGradX, 3, 3, 2>(p, tiles, ncols, s);
        if (rc != ATB_OK) return rc;
    }
    if (need_w) {
        const int ncols = O <= 64 ? 64 : 128;
        const int mt = ceil_div(K, TcM), nt = ceil_div(O, ncols);
        const long long tiles_mn = static_cast<long long>(mt) * nt;
        const long long gz = z.gz;
#define ATB_TC_PW(DT)                                                                                                     \
    {                                                                                                                     \
        PkGradW<DT> p{};                                                                                                  \
        p.x = x; p.dw = dw; p.gwp = gwp; p.gw = grad_w; p.part = part; p.O = O; p.K = K; p.pad_index = pad_index;         \
        p.gz = static_cast<int>(gz);                                                                                      \
        p.P = z.P; p.Ppad = z.Ppad; p.gw_plane = static_cast<long long>(O) * z.Ppad; p.g = g;                             \
        p.divL = tc_fastdiv(L); p.divOW = tc_fastdiv(g.OW); p.divKK = tc_fastdiv(KK); p.divKW = tc_fastdiv(g.KW);          \
        p.mt = mt; p.nt = nt; p.divKH = tc_fastdiv(g.KH);                                                                 \
        p.window = (g.SW == 1 && g.DW == 1 && (g.KW == 2 || g.KW == 3)) ? 1 : 0;                                          \
        rc = exact_tables ? tc_packed_launch<PkGradW<DT>, 1, 3, 3>(p, tiles_mn * gz, ncols, s)                            \
                          : tc_packed_launch<PkGradW<DT>, 3, 3, 2>(p, tiles_mn * gz, ncols, s);                            \
    }
        int rc = ATB_OK;
        if (x_dtype == ATB_U8) ATB_TC_PW(ATB_U8)
        else if (x_dtype == ATB_I8) ATB_TC_PW(ATB_I8)
        else ATB_TC_PW(ATB_F32)
#undef ATB_TC_PW
        if (rc != ATB_OK) return rc;
        if (part != nullptr) {
            const long long n = static_cast<long long>(O) * K;
            tc_sum_slices_kernel<<<grid_for(n, 256, 4096), 256, 0, s>>>(part, grad_w, z.gz_used, n);
            return check_launch("tc_sum_slices_kernel");
        }
    }
    return ATB_OK;
}

int tc_status_read(int* status)
{
    cudaError_t e = cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int));
    if (e != cudaSuccess) { set_error("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    return ATB_OK;
}

}  // namespace atb
