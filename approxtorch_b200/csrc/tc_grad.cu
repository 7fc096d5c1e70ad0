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

int tc_status_read(int* status)
{
    cudaError_t e = cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int));
    if (e != cudaSuccess) { set_error("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    return ATB_OK;
}

}  // namespace atb
