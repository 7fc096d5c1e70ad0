// STE / LRE backward: dense fp32 contractions whose operands are 256-entry table maps of the saved
// 8-bit tensors.  The maps, the im2col gather and the fold are fused into the operand fetch of one
// tiled fp32 GEMM kernel (128 x 128 x 8 tiles, 8 x 8 outputs per thread), so neither the mapped
// operand X' = dw[idx(x)] nor the column matrix is ever written to memory
// (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:443-524 materialises X' for cuBLAS;
// approxtorch/nn/bgemm_int8.py:165-212, 259-295 hands the image form to cuDNN).
//
//   grad_x[n,k,l] = sum_o go[n,o,l] * dx[idx(w[o,k])]        grad_w[o,k] = sum_{n,l} go[n,o,l] * dw[idx(x[n,k,l])]
//
// fp32 FMA throughout (no TF32): these gradients carry a rel-1e-5 bar.  grad_w reduces over all
// pixels, so its launch is split over the pixel axis and the partial tiles are added with fp32
// atomics into a zeroed output.
#include "common.cuh"

namespace atb {

struct FastDiv {
    unsigned d, mul, shift;
};

static FastDiv make_fastdiv(unsigned d)
{
    FastDiv f;
    f.d = d < 1 ? 1 : d;
    unsigned s = 0;
    while ((1ull << s) < f.d) ++s;
    f.shift = s;
    f.mul = static_cast<unsigned>((((1ull << s) - f.d) << 32) / f.d + 1);
    return f;
}

// valid for n < 2^31
__device__ __forceinline__ unsigned fdiv(unsigned n, const FastDiv& f)
{
    return (__umulhi(n, f.mul) + n) >> f.shift;
}

__device__ __forceinline__ int index_rt(const void* base, long long i, int dtype)
{
    if (dtype == ATB_U8) return index_of<ATB_U8>(base, i);
    if (dtype == ATB_I8) return index_of<ATB_I8>(base, i);
    return index_of<ATB_F32>(base, i);
}

constexpr int TK = 8;        // contraction slice per shared-memory stage

// ------------------------------------------------------------------------------------------------
// problem descriptions: a(m, r), b(r, n), store(m, n, v)
// ------------------------------------------------------------------------------------------------

// Operand fetch of one thread for one 128 x 8 slice of A and of B: slot q covers element e = tid + 256 q.
// kARFast / kBRFast say which index runs fastest over the threads (the one that is contiguous in memory).
// Problems whose index arithmetic is cheap use this generic form; the conv problems bring their own, which
// hoists everything that does not change from slice to slice.
template <class Prob>
__device__ __forceinline__ void generic_fetch(const Prob& p, int tid, int m0, int n0, int r0, int rend,
                                              float (&ra)[4], float (&rb)[4])
{
    const int M = p.M(), N = p.N();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int e = tid + 256 * q;
        const int ml = Prob::kARFast ? (e >> 3) : (e & 127);
        const int rl = Prob::kARFast ? (e & 7) : (e >> 7);
        const int m = m0 + ml, r = r0 + rl;
        ra[q] = (m < M && r < rend) ? p.a(m, r) : 0.0f;
        const int nl = Prob::kBRFast ? (e >> 3) : (e & 127);
        const int sl = Prob::kBRFast ? (e & 7) : (e >> 7);
        const int n = n0 + nl, sr = r0 + sl;
        rb[q] = (n < N && sr < rend) ? p.b(sr, n) : 0.0f;
    }
}

// column space, grad_x of batch item z:  C[k, l] = sum_o dx[idx(w[o,k])] * go[z, o, l]
struct ColGradX {
    const float* go; const void* w; int w_dtype; int w_ok; const float* dx; float* gx;
    int K, L, O;
    long long z;
    static constexpr bool kAtomic = false, kARFast = false, kBRFast = false;
    __device__ int M() const { return K; }
    __device__ int N() const { return L; }
    __device__ void setup(int zz, int nz, int& rbeg, int& rend) { z = zz; rbeg = 0; rend = O; }
    __device__ float a(int k, int o) const
    {
        const long long i = w_ok ? static_cast<long long>(o) * K + k : static_cast<long long>(k) * O + o;
        return __ldg(dx + index_rt(w, i, w_dtype));
    }
    __device__ float b(int o, int l) const { return __ldg(go + (z * O + o) * L + l); }
    __device__ void store(int k, int l, float v) const { gx[(z * K + k) * L + l] = v; }
    __device__ void prep(int, int, int) {}
    __device__ void fetch(int tid, int m0, int n0, int r0, int rend, float (&ra)[4], float (&rb)[4]) const
    {
        generic_fetch(*this, tid, m0, n0, r0, rend, ra, rb);
    }
};

// column space, grad_w:  C[o, k] = sum_{p=(n,l)} go[n,o,l] * dw[idx(x[n,k,l])]
struct ColGradW {
    const float* go; const void* x; int x_dtype; const float* dw; float* gw; int w_ok;
    int K, L, O; long long P;
    FastDiv divL;
    static constexpr bool kAtomic = true, kARFast = true, kBRFast = true;
    __device__ int M() const { return O; }
    __device__ int N() const { return K; }
    __device__ void setup(int zz, int nz, int& rbeg, int& rend)
    {
        const long long per = ((P + nz - 1) / nz + TK - 1) / TK * TK;
        const long long b0 = per * zz;
        rbeg = static_cast<int>(b0 < P ? b0 : P);
        rend = static_cast<int>(b0 + per < P ? b0 + per : P);
    }
    __device__ float a(int o, int p) const
    {
        const unsigned n = fdiv(p, divL);
        const unsigned l = p - n * L;
        return __ldg(go + (static_cast<long long>(n) * O + o) * L + l);
    }
    __device__ float b(int p, int k) const
    {
        const unsigned n = fdiv(p, divL);
        const unsigned l = p - n * L;
        return __ldg(dw + index_rt(x, (static_cast<long long>(n) * K + k) * L + l, x_dtype));
    }
    __device__ void store(int o, int k, float v) const
    {
        atomicAdd(gw + (w_ok ? static_cast<long long>(o) * K + k : static_cast<long long>(k) * O + o), v);
    }
    __device__ void prep(int, int, int) {}
    __device__ void fetch(int tid, int m0, int n0, int r0, int rend, float (&ra)[4], float (&rb)[4]) const
    {
        generic_fetch(*this, tid, m0, n0, r0, rend, ra, rb);
    }
};

// image space, grad_x:  C[m=(n,h,w), c] = sum_{r=(o,i,j)} go[n,o,oh,ow] * gs[o] * dx[widx[o,(c,i,j)]]
struct ConvGradX {
    const float* go; const uint8_t* widx; const float* dx; const float* gs; const float* wz; float* gx;
    int Nb, O, K; ConvGeom g;
    FastDiv divHW, divW, divKK, divKW, divSH, divSW;
    const uint8_t* xmask; const float* xscale;      // optional: fake-quant backward (mask ? v : 0) / max(scale, 1e-12) in the store
    static constexpr bool kAtomic = false, kARFast = false, kBRFast = false;
    __device__ int M() const { return Nb * g.H * g.W; }
    __device__ int N() const { return g.C; }
    __device__ void setup(int zz, int nz, int& rbeg, int& rend) { rbeg = 0; rend = O * g.KH * g.KW; }
    __device__ float a(int m, int r) const
    {
        const unsigned n = fdiv(m, divHW);
        const unsigned hw = m - n * (g.H * g.W);
        const unsigned h = fdiv(hw, divW);
        const unsigned w = hw - h * g.W;
        const unsigned o = fdiv(r, divKK);
        const unsigned ij = r - o * (g.KH * g.KW);
        const unsigned i = fdiv(ij, divKW);
        const unsigned j = ij - i * g.KW;
        const int th = static_cast<int>(h) + g.PH - static_cast<int>(i) * g.DH;
        const int tw = static_cast<int>(w) + g.PW - static_cast<int>(j) * g.DW;
        if (th < 0 || tw < 0) return 0.0f;
        const unsigned oh = fdiv(th, divSH), ow = fdiv(tw, divSW);
        if (oh * g.SH != static_cast<unsigned>(th) || ow * g.SW != static_cast<unsigned>(tw)) return 0.0f;
        if (oh >= static_cast<unsigned>(g.OH) || ow >= static_cast<unsigned>(g.OW)) return 0.0f;
        return __ldg(go + ((static_cast<long long>(n) * O + o) * g.OH + oh) * g.OW + ow);
    }
    __device__ float b(int r, int c) const
    {
        const unsigned o = fdiv(r, divKK);
        const unsigned ij = r - o * (g.KH * g.KW);
        float v = __ldg(dx + __ldg(widx + static_cast<long long>(o) * K + c * (g.KH * g.KW) + ij));
        if (wz != nullptr) v -= __ldg(wz + o);
        if (gs != nullptr) v *= __ldg(gs + o);
        return v;
    }
    __device__ void store(int m, int c, float v) const
    {
        const unsigned n = fdiv(m, divHW);
        const unsigned hw = m - n * (g.H * g.W);
        const long long at = (static_cast<long long>(n) * g.C + c) * (g.H * g.W) + hw;
        if (xmask != nullptr) v = (xmask[at] ? v : 0.0f) / fmaxf(__ldg(xscale), 1e-12f);
        gx[at] = v;
    }
    // Every thread fetches for ONE image pixel m and ONE input channel c (element e = tid + 256 q has
    // m = m0 + (tid & 127), r = r0 + (tid >> 7) + 2 q), so the pixel's decomposition is done once per block tile
    // and the (o, i, j) decomposition of r once per slot, shared by the A and the B element.
    const float* go_n;        // &go[n, 0, 0, 0] of this thread's pixel
    int hp, wp;               // h + PH, w + PW (or a large negative value when m is past the end)
    int ckk;                  // c * KH * KW, or -1 when c is past the end
    __device__ void prep(int tid, int m0, int n0)
    {
        const int m = m0 + (tid & 127);
        hp = wp = -(1 << 28);
        go_n = go;
        if (m < M()) {
            const unsigned n = fdiv(m, divHW);
            const unsigned hw = m - n * (g.H * g.W);
            const unsigned h = fdiv(hw, divW);
            hp = static_cast<int>(h) + g.PH;
            wp = static_cast<int>(hw - h * g.W) + g.PW;
            go_n = go + static_cast<long long>(n) * O * g.OH * g.OW;
        }
        const int c = n0 + (tid & 127);
        ckk = c < g.C ? c * (g.KH * g.KW) : -1;
    }
    __device__ void fetch(int tid, int, int, int r0, int rend, float (&ra)[4], float (&rb)[4]) const
    {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int r = r0 + (tid >> 7) + 2 * q;
            float av = 0.0f, bv = 0.0f;
            if (r < rend) {
                const unsigned o = fdiv(r, divKK);
                const unsigned ij = r - o * (g.KH * g.KW);
                const unsigned i = fdiv(ij, divKW);
                const unsigned j = ij - i * g.KW;
                const int th = hp - static_cast<int>(i) * g.DH;
                const int tw = wp - static_cast<int>(j) * g.DW;
                if (th >= 0 && tw >= 0) {
                    unsigned oh = th, ow = tw;
                    bool hit = true;
                    if (g.SH != 1 || g.SW != 1) {
                        oh = fdiv(th, divSH); ow = fdiv(tw, divSW);
                        hit = oh * g.SH == static_cast<unsigned>(th) && ow * g.SW == static_cast<unsigned>(tw);
                    }
                    if (hit && oh < static_cast<unsigned>(g.OH) && ow < static_cast<unsigned>(g.OW))
                        av = __ldg(go_n + (static_cast<long long>(o) * g.OH + oh) * g.OW + ow);
                }
                if (ckk >= 0) {
                    bv = __ldg(dx + __ldg(widx + static_cast<long long>(o) * K + ckk + ij));
                    if (wz != nullptr) bv -= __ldg(wz + o);
                    if (gs != nullptr) bv *= __ldg(gs + o);
                }
            }
            ra[q] = av;
            rb[q] = bv;
        }
    }
};

// image space, grad_w:  C[o, k=(c,i,j)] = gs[o] * sum_{p=(n,oh,ow)} go[n,o,oh,ow] * dw[idx(x[n,c,ih,iw]) or pad]
struct ConvGradW {
    const float* go; const void* x; int x_dtype; const float* dw; const float* gs; float* gw;
    int O, K, pad_index; long long P; ConvGeom g;
    FastDiv divL, divOW, divKK, divKW;
    static constexpr bool kAtomic = true, kARFast = true, kBRFast = true;
    __device__ int M() const { return O; }
    __device__ int N() const { return K; }
    __device__ void setup(int zz, int nz, int& rbeg, int& rend)
    {
        const long long per = ((P + nz - 1) / nz + TK - 1) / TK * TK;
        const long long b0 = per * zz;
        rbeg = static_cast<int>(b0 < P ? b0 : P);
        rend = static_cast<int>(b0 + per < P ? b0 + per : P);
    }
    __device__ float a(int o, int p) const
    {
        const unsigned n = fdiv(p, divL);
        const unsigned l = p - n * (g.OH * g.OW);
        return __ldg(go + (static_cast<long long>(n) * O + o) * (g.OH * g.OW) + l);
    }
    __device__ float b(int p, int k) const
    {
        const unsigned n = fdiv(p, divL);
        const unsigned l = p - n * (g.OH * g.OW);
        const unsigned oh = fdiv(l, divOW);
        const unsigned ow = l - oh * g.OW;
        const unsigned c = fdiv(k, divKK);
        const unsigned ij = k - c * (g.KH * g.KW);
        const unsigned i = fdiv(ij, divKW);
        const unsigned j = ij - i * g.KW;
        const int ih = static_cast<int>(oh) * g.SH - g.PH + static_cast<int>(i) * g.DH;
        const int iw = static_cast<int>(ow) * g.SW - g.PW + static_cast<int>(j) * g.DW;
        int idx = pad_index;
        if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
            idx = index_rt(x, ((static_cast<long long>(n) * g.C + c) * g.H + ih) * g.W + iw, x_dtype);
        return __ldg(dw + idx);
    }
    __device__ void store(int o, int k, float v) const
    {
        if (gs != nullptr) v *= __ldg(gs + o);
        atomicAdd(gw + static_cast<long long>(o) * K + k, v);
    }
    // Every thread fetches for ONE output pixel p = r0 + (tid & 7) per slice and for four fixed channels
    // o = m0 + (tid >> 3) + 32 q and four fixed taps k = n0 + (tid >> 3) + 32 q: the tap decompositions are done
    // once per block tile, the pixel decomposition once per slice.
    int o_off[4];             // o * OH * OW, or -1 when o is past the end
    int k_off[4];             // (c * H + (i*DH - PH)) * W + (j*DW - PW): offset of the tap from the pixel's window origin
    short k_dh[4], k_dw[4];   // i*DH - PH, j*DW - PW; k_dh = -32768 when k is past the end
    __device__ void prep(int tid, int m0, int n0)
    {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int o = m0 + (tid >> 3) + 32 * q;
            o_off[q] = o < O ? o * (g.OH * g.OW) : -1;
            const int k = n0 + (tid >> 3) + 32 * q;
            k_off[q] = 0; k_dh[q] = -32768; k_dw[q] = 0;
            if (k < K) {
                const unsigned c = fdiv(k, divKK);
                const unsigned ij = k - c * (g.KH * g.KW);
                const unsigned i = fdiv(ij, divKW);
                const unsigned j = ij - i * g.KW;
                const int dh = static_cast<int>(i) * g.DH - g.PH, dw_ = static_cast<int>(j) * g.DW - g.PW;
                k_dh[q] = static_cast<short>(dh); k_dw[q] = static_cast<short>(dw_);
                k_off[q] = (static_cast<int>(c) * g.H + dh) * g.W + dw_;
            }
        }
    }
    __device__ void fetch(int tid, int, int, int r0, int rend, float (&ra)[4], float (&rb)[4]) const
    {
        const int pp = r0 + (tid & 7);
        if (pp >= rend) {
#pragma unroll
            for (int q = 0; q < 4; ++q) { ra[q] = 0.0f; rb[q] = 0.0f; }
            return;
        }
        const unsigned n = fdiv(pp, divL);
        const unsigned l = pp - n * (g.OH * g.OW);
        const unsigned oh = fdiv(l, divOW);
        const int ih0 = static_cast<int>(oh) * g.SH, iw0 = static_cast<int>(l - oh * g.OW) * g.SW;
        const float* go_p = go + static_cast<long long>(n) * O * (g.OH * g.OW) + l;
        const long long x_p = static_cast<long long>(n) * g.C * g.H * g.W + static_cast<long long>(ih0) * g.W + iw0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            ra[q] = o_off[q] >= 0 ? __ldg(go_p + o_off[q]) : 0.0f;
            float bv = 0.0f;
            if (k_dh[q] != -32768) {
                const int ih = ih0 + k_dh[q], iw = iw0 + k_dw[q];
                int idx = pad_index;
                if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
                    idx = index_rt(x, x_p + k_off[q], x_dtype);
                bv = __ldg(dw + idx);
            }
            rb[q] = bv;
        }
    }
};


// ------------------------------------------------------------------------------------------------
// Lean conv problems (32-bit offsets, branch-free operand fetch).  Used whenever every tensor has fewer
// than 2^31 elements and the kernel window has at most 128 taps; the two descriptions above stay as the
// general fallback.
// ------------------------------------------------------------------------------------------------
constexpr int kMaxTaps = 128;

// image space, grad_x, tap-major and split by stride class.
// A pixel (h, w) only receives from taps with (h + PH - i*DH) % SH == 0 and (w + PW - j*DW) % SW == 0, so the
// pixels are grouped by class (a, b) = ((h + PH) % SH, (w + PW) % SW) = blockIdx.z and every block runs over
// the taps of its class only: with stride 2 a 3 x 3 window costs 9/4 tap-passes per pixel instead of 9.
// The contraction index runs tap-major, r = tap * O8 + o (O8 = O rounded up to the slice length), so one
// slice of 8 belongs to one tap and the window arithmetic is done once per slice, not once per element.
struct ConvGradXTaps {
    const float* go; const uint8_t* widx; const float* dx; const float* gs; const float* wz; float* gx;
    int Nb, O, K, O8; ConvGeom g;
    FastDiv divSH, divSW;
    const uint8_t* xmask; const float* xscale;      // optional fake-quant backward in the store
    static constexpr bool kAtomic = false, kARFast = false, kBRFast = false;
    // block state
    int Mc, Hc, Wc, h0, w0, ntaps;
    // thread state
    int hp, wp, go_n, ckk, tap, o0;
    __device__ int M() const { return Mc; }
    __device__ int N() const { return g.C; }
    __device__ void setup(int zz, int, int& rbeg, int& rend)
    {
        __shared__ int s_dh[kMaxTaps], s_dw[kMaxTaps], s_ij[kMaxTaps], s_n;
        const int a = zz / g.SW, b = zz - a * g.SW;
        h0 = ((a - g.PH) % g.SH + g.SH) % g.SH;            // first row of the class
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
    const int* tap_dh; const int* tap_dw; const int* tap_ij;
    __device__ void pixel_of(int m, int& n, int& h, int& w) const
    {
        const int hw = Hc * Wc;
        n = m / hw;
        const int rem = m - n * hw;
        const int t = rem / Wc;
        h = h0 + g.SH * t;
        w = w0 + g.SW * (rem - t * Wc);
    }
    __device__ void prep(int tid, int m0, int n0)
    {
        const int m = m0 + (tid & 127);
        hp = wp = -(1 << 28);
        go_n = 0;
        if (m < Mc) {
            int n, h, w;
            pixel_of(m, n, h, w);
            hp = h + g.PH; wp = w + g.PW;
            go_n = n * O * g.OH * g.OW;
        }
        const int c = n0 + (tid & 127);
        ckk = c < g.C ? c * (g.KH * g.KW) : -1;
        tap = 0; o0 = 0;
    }
    // called for consecutive slices r0 = 0, 8, 16, ...
    __device__ void fetch(int tid, int, int, int, int, float (&ra)[4], float (&rb)[4])
    {
        const int th = hp - tap_dh[tap], tw = wp - tap_dw[tap], ij = tap_ij[tap];
        unsigned oh = th, ow = tw;
        if (g.SH != 1) oh = fdiv(th < 0 ? 0 : th, divSH);
        if (g.SW != 1) ow = fdiv(tw < 0 ? 0 : tw, divSW);
        const bool hit = th >= 0 && tw >= 0 && oh < static_cast<unsigned>(g.OH) && ow < static_cast<unsigned>(g.OW);
        const int a_off = hit ? go_n + static_cast<int>(oh) * g.OW + static_cast<int>(ow) : 0;
        const int ohw = g.OH * g.OW;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int o = o0 + (tid >> 7) + 2 * q;
            const bool o_ok = o < O;
            const float av = __ldg(go + (hit && o_ok ? a_off + o * ohw : 0));
            ra[q] = hit && o_ok ? av : 0.0f;
            const bool b_ok = o_ok && ckk >= 0;
            const int wi = __ldg(widx + (b_ok ? o * K + ckk + ij : 0));
            float bv = __ldg(dx + wi);
            if (wz != nullptr) bv -= __ldg(wz + (o_ok ? o : 0));
            if (gs != nullptr) bv *= __ldg(gs + (o_ok ? o : 0));
            rb[q] = b_ok ? bv : 0.0f;
        }
        o0 += TK;
        if (o0 >= O8) { o0 = 0; ++tap; }
    }
    __device__ void store(int m, int c, float v) const
    {
        int n, h, w;
        pixel_of(m, n, h, w);
        const int at = ((n * g.C + c) * g.H + h) * g.W + w;
        if (xmask != nullptr) v = (xmask[at] ? v : 0.0f) / fmaxf(__ldg(xscale), 1e-12f);
        gx[at] = v;
    }
};

// image space, grad_w with the pixel decomposition done once per slice, 32-bit offsets and the operand type
// of the saved image fixed at compile time.
template <int XDT>
struct ConvGradWLean {
    const float* go; const void* x; const float* dw; const float* gs; float* gw;
    int O, K, pad_index; long long P; ConvGeom g;
    FastDiv divL, divOW, divKK, divKW;
    static constexpr bool kAtomic = true, kARFast = true, kBRFast = true;
    int o_off[4], k_off[4], k_dhw[4];       // k_dhw: (i*DH - PH) in the high half, (j*DW - PW) in the low half
    unsigned ok_mask;                       // bit q: channel slot q valid; bit 4 + q: tap slot q valid
    __device__ int M() const { return O; }
    __device__ int N() const { return K; }
    __device__ void setup(int zz, int nz, int& rbeg, int& rend)
    {
        const long long per = ((P + nz - 1) / nz + TK - 1) / TK * TK;
        const long long b0 = per * zz;
        rbeg = static_cast<int>(b0 < P ? b0 : P);
        rend = static_cast<int>(b0 + per < P ? b0 + per : P);
    }
    __device__ void prep(int tid, int m0, int n0)
    {
        ok_mask = 0u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int o = m0 + (tid >> 3) + 32 * q;
            o_off[q] = o < O ? o * (g.OH * g.OW) : 0;
            if (o < O) ok_mask |= 1u << q;
            const int k = n0 + (tid >> 3) + 32 * q;
            k_off[q] = 0; k_dhw[q] = 0;
            if (k < K) {
                const unsigned c = fdiv(k, divKK);
                const unsigned ij = k - c * (g.KH * g.KW);
                const unsigned i = fdiv(ij, divKW);
                const unsigned j = ij - i * g.KW;
                const int dh = static_cast<int>(i) * g.DH - g.PH, dw_ = static_cast<int>(j) * g.DW - g.PW;
                k_dhw[q] = (dh << 16) | (dw_ & 0xffff);
                k_off[q] = (static_cast<int>(c) * g.H + dh) * g.W + dw_;
                ok_mask |= 16u << q;
            }
        }
    }
    __device__ void fetch(int tid, int, int, int r0, int rend, float (&ra)[4], float (&rb)[4]) const
    {
        const int pp = r0 + (tid & 7);
        const bool p_ok = pp < rend;
        const unsigned pc = p_ok ? pp : 0;
        const unsigned n = fdiv(pc, divL);
        const unsigned l = pc - n * (g.OH * g.OW);
        const unsigned oh = fdiv(l, divOW);
        const int ih0 = static_cast<int>(oh) * g.SH, iw0 = static_cast<int>(l - oh * g.OW) * g.SW;
        const int go_off = static_cast<int>(n) * O * (g.OH * g.OW) + static_cast<int>(l);
        const int x_off = (static_cast<int>(n) * g.C * g.H + ih0) * g.W + iw0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bool a_ok = p_ok && ((ok_mask >> q) & 1u);
            const float av = __ldg(go + (a_ok ? go_off + o_off[q] : 0));
            ra[q] = a_ok ? av : 0.0f;
            const bool b_ok = p_ok && ((ok_mask >> (4 + q)) & 1u);
            const int ih = ih0 + (k_dhw[q] >> 16), iw = iw0 + static_cast<short>(k_dhw[q] & 0xffff);
            const bool inside = b_ok && static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) &&
                                static_cast<unsigned>(iw) < static_cast<unsigned>(g.W);
            const int xi = index_of<XDT>(x, inside ? x_off + k_off[q] : 0);
            const float bv = __ldg(dw + (inside ? xi : pad_index));
            rb[q] = b_ok ? bv : 0.0f;
        }
    }
    __device__ void store(int o, int k, float v) const
    {
        if (gs != nullptr) v *= __ldg(gs + o);
        atomicAdd(gw + o * K + k, v);
    }
};

// ------------------------------------------------------------------------------------------------
// the tiled kernel
// ------------------------------------------------------------------------------------------------
// TMv x TNv outputs per block (128 or 64 each): 16 x 16 threads, (TMv / 16) x (TNv / 16) outputs per thread.  The
// operand fetch always covers 128 rows / columns; with a 64-wide tile the upper half is not kept (the
// problems mask it out anyway when M or N is at most 64, which is when the launcher picks the narrow tile).
template <class Prob, int TMv, int TNv>
__global__ void __launch_bounds__(256, 2) fused_sgemm_kernel(const Prob prob_in)
{
    static_assert((TMv == 64 || TMv == 128) && (TNv == 64 || TNv == 128), "tile sides are 64 or 128");
    constexpr int RM = TMv / 16, RN = TNv / 16;
    __shared__ __align__(16) float As[2][TK][TMv + 4];
    __shared__ __align__(16) float Bs[2][TK][TNv + 4];
    Prob p = prob_in;
    int rbeg, rend;
    p.setup(blockIdx.z, gridDim.z, rbeg, rend);
    const int M = p.M(), N = p.N();
    if (static_cast<int>(blockIdx.x) * TMv >= M) return;        // stride classes differ in size: surplus blocks leave
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * TMv, n0 = blockIdx.y * TNv;
    const int tx = tid & 15, ty = tid >> 4;

    float acc[RM][RN];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < RN; ++j) acc[i][j] = 0.0f;
    if (rbeg >= rend) {
        if (Prob::kAtomic) return;     // nothing to add
    }

    float ra[4], rb[4];
    p.prep(tid, m0, n0);
    auto fetch = [&](int r0) { p.fetch(tid, m0, n0, r0, rend, ra, rb); };
    auto stash = [&](int buf) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = tid + 256 * q;
            const int ml = Prob::kARFast ? (e >> 3) : (e & 127);
            const int rl = Prob::kARFast ? (e & 7) : (e >> 7);
            if (TMv == 128 || ml < TMv) As[buf][rl][ml] = ra[q];
            const int nl = Prob::kBRFast ? (e >> 3) : (e & 127);
            const int sl = Prob::kBRFast ? (e & 7) : (e >> 7);
            if (TNv == 128 || nl < TNv) Bs[buf][sl][nl] = rb[q];
        }
    };

    const int ntiles = (rend - rbeg + TK - 1) / TK;
    if (ntiles > 0) { fetch(rbeg); stash(0); }
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        if (t + 1 < ntiles) fetch(rbeg + (t + 1) * TK);
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float av[RM], bv[RN];
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
            if constexpr (RM == 8) {
                const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
                av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
            }
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
            if constexpr (RN == 8) {
                const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
                bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
            }
#pragma unroll
            for (int i = 0; i < RM; ++i)
#pragma unroll
                for (int j = 0; j < RN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (t + 1 < ntiles) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < RN; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n < N) p.store(m, n, acc[i][j]);
        }
    }
}

static long long sgemm_tiles(long long M, long long N)
{
    return ((M + (M <= 64 ? 63 : 127)) / (M <= 64 ? 64 : 128)) * ((N + (N <= 64 ? 63 : 127)) / (N <= 64 ? 64 : 128));
}

// narrow tiles when the whole M (or N) extent fits in 64
template <class Prob>
static void launch_sgemm(const Prob& p, long long M, long long N, unsigned gz, cudaStream_t s)
{
    const bool m64 = M <= 64, n64 = N <= 64;
    dim3 grid(ceil_div(M, m64 ? 64 : 128), ceil_div(N, n64 ? 64 : 128), gz);
    if (m64 && n64) fused_sgemm_kernel<Prob, 64, 64><<<grid, 256, 0, s>>>(p);
    else if (m64) fused_sgemm_kernel<Prob, 64, 128><<<grid, 256, 0, s>>>(p);
    else if (n64) fused_sgemm_kernel<Prob, 128, 64><<<grid, 256, 0, s>>>(p);
    else fused_sgemm_kernel<Prob, 128, 128><<<grid, 256, 0, s>>>(p);
}

__global__ void zero_kernel(float* p, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = 0.0f;
}

static int split_factor(long long tiles, long long P)
{
    const int target = 3 * sm_count();
    long long s = tiles >= target ? 1 : (target + tiles - 1) / tiles;
    const long long maxs = (P + 4 * TK - 1) / (4 * TK);
    if (s > maxs) s = maxs;
    if (s > 1024) s = 1024;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

}  // namespace atb

using namespace atb;

extern "C" size_t atb_lre_conv_bwd_scratch_bytes(int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw, int ph, int pw,
                                                 int dh, int dw_, int flags, int need_x, int need_w)
{
    int OH = 0, OW = 0;
    if (N <= 0 || C <= 0 || O <= 0 || N > 65535 || (flags & 6) != 0 || (!need_x && !need_w)) return 0;
    if (!conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw_, &OH, &OW)) return 0;
    if (static_cast<long long>(sh) * sw > 64 || static_cast<long long>(kh) * kw > 128) return 0;
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw_, OH, OW};
    return tc_packed_scratch_bytes(N, O, g, need_x != 0, need_w != 0, (flags & 1) != 0, (flags & 8) != 0);
}

extern "C" int atb_tensor_core_status(int* status /*host*/)
{
    ATB_REQUIRE(status != nullptr, "status is null");
    return tc_status_read(status);
}

extern "C" int atb_lre_bwd(const float* go, const void* x, int x_dtype, const void* w, int w_dtype, int w_ok_layout,
                           const float* dx, const float* dw, float* grad_x, float* grad_w,
                           int N, int K, int L, int O, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    ATB_REQUIRE(x_dtype >= 0 && x_dtype <= 2 && w_dtype >= 0 && w_dtype <= 2, "bad dtype");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long P = static_cast<long long>(N) * L;
    ATB_REQUIRE(P < 2147483647LL, "N*L too large");
    int rc = ATB_OK;
    if (grad_x != nullptr && P * K > 0) {
        if (O == 0) {
            zero_kernel<<<grid_for(P * K, 256, 4096), 256, 0, s>>>(grad_x, P * K);
        } else {
            ATB_REQUIRE(go && w && dx, "null pointer");
            ATB_REQUIRE(N <= 65535, "batch above 65535 is not supported");
            ColGradX p{go, w, w_dtype, w_ok_layout, dx, grad_x, K, L, O, 0};
            ATB_REQUIRE(ceil_div(L, 64) <= 65535, "L too large");
            launch_sgemm(p, K, L, N, s);
        }
        rc = check_launch("lre grad_x");
        if (rc != ATB_OK) return rc;
    }
    if (grad_w != nullptr && static_cast<long long>(O) * K > 0) {
        zero_kernel<<<grid_for(static_cast<long long>(O) * K, 256, 4096), 256, 0, s>>>(grad_w, static_cast<long long>(O) * K);
        rc = check_launch("zero_kernel");
        if (rc != ATB_OK) return rc;
        if (P > 0) {
            ATB_REQUIRE(go && x && dw, "null pointer");
            ColGradW p{go, x, x_dtype, dw, grad_w, w_ok_layout, K, L, O, P, make_fastdiv(L)};
            ATB_REQUIRE(ceil_div(K, 64) <= 65535, "K too large");
            launch_sgemm(p, O, K, split_factor(sgemm_tiles(O, K), P), s);
            rc = check_launch("lre grad_w");
        }
    }
    return rc;
}

extern "C" int atb_lre_conv_bwd(const float* go, const void* x, int x_dtype, const uint8_t* widx,
                                const float* dx, const float* dw, const float* go_scale, const float* w_zero,
                                const uint8_t* x_mask, const float* x_scale,
                                float* grad_x, float* grad_w,
                                int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw, int ph, int pw,
                                int dh, int dw_, int pad_index, int flags, void* scratch, size_t scratch_bytes, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0 && O >= 0, "negative dimension");
    ATB_REQUIRE(x_dtype >= 0 && x_dtype <= 2, "bad dtype");
    ATB_REQUIRE(pad_index >= 0 && pad_index <= 256, "pad_index out of range");
    ATB_REQUIRE((x_mask == nullptr) == (x_scale == nullptr), "x_mask and x_scale go together");
    const bool exact_tables = (flags & 1) != 0;      // dx / dw (and w_zero) hold integers of magnitude <= 256
    const bool simt_only = (flags & 2) != 0;         // keep to the fp32 SIMT kernels
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw_, &OH, &OW), "conv geometry yields empty output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw_, OH, OW};
    const long long K = static_cast<long long>(C) * kh * kw;
    const long long Mx = static_cast<long long>(N) * H * W;
    const long long P = static_cast<long long>(N) * OH * OW;
    ATB_REQUIRE(Mx < 2147483647LL && P < 2147483647LL && K < 2147483647LL &&
                static_cast<long long>(O) * kh * kw < 2147483647LL &&
                static_cast<long long>(C) * H * W < 2147483647LL && static_cast<long long>(O) * OH * OW < 2147483647LL,
                "dimensions too large");
    ATB_REQUIRE(static_cast<long long>(kh) * dh < 30000 && static_cast<long long>(kw) * dw_ < 30000 && ph < 30000 && pw < 30000,
                "kernel extent or padding too large");
    // every tensor addressable with 32-bit offsets and a window the tap table can hold: the lean problems apply
    const bool lean = static_cast<long long>(N) * O * OH * OW < 2147483647LL && Mx * C < 2147483647LL &&
                      static_cast<long long>(O) * K < 2147483647LL && kh * kw <= kMaxTaps;
    int rc = ATB_OK;
    // Operands packed ahead of the contraction when the caller brought enough scratch for it.
    const bool want_x = grad_x != nullptr && Mx * C > 0, want_w = grad_w != nullptr && O * K > 0;
    if (lean && !simt_only && (flags & 4) == 0 && scratch != nullptr && O > 0 && P > 0 && N <= 65535 && (want_x || want_w) &&
        sh * sw <= 64 && kh * kw <= 128) {
        const bool deterministic = (flags & 8) != 0;
        const size_t need = tc_packed_scratch_bytes(N, O, g, want_x, want_w, exact_tables, deterministic);
        if (need > 0 && scratch_bytes >= need) {
            ATB_REQUIRE(aligned_to(scratch, 16), "scratch must be 16-byte aligned");
            ATB_REQUIRE(go && (!want_x || (widx && dx)) && (!want_w || (x && dw)), "null pointer");
            if (want_w) {
                zero_kernel<<<grid_for(O * K, 256, 4096), 256, 0, s>>>(grad_w, O * K);
                rc = check_launch("zero_kernel");
                if (rc != ATB_OK) return rc;
            }
            return tc_packed_conv_bwd(go, x, x_dtype, widx, dx, dw, go_scale, w_zero, x_mask, x_scale, want_x ? grad_x : nullptr,
                                      want_w ? grad_w : nullptr, N, O, g, pad_index, exact_tables, deterministic, scratch, s);
        }
    }
    if (grad_x != nullptr && Mx * C > 0) {
        if (O == 0) {
            zero_kernel<<<grid_for(Mx * C, 256, 4096), 256, 0, s>>>(grad_x, Mx * C);
        } else {
            ATB_REQUIRE(go && widx && dx, "null pointer");
            if (lean && !simt_only && sh * sw <= 64 && kh * kw <= 128) {
                rc = tc_conv_grad_x(go, widx, dx, go_scale, w_zero, x_mask, x_scale, grad_x, N, O, g, exact_tables, s);
                if (rc != ATB_OK) return rc;
            } else if (lean && sh * sw <= 64) {
                ConvGradXTaps p{go, widx, dx, go_scale, w_zero, grad_x, N, O, static_cast<int>(K), (O + TK - 1) / TK * TK, g,
                                make_fastdiv(sh), make_fastdiv(sw), x_mask, x_scale};
                const long long max_class = static_cast<long long>(N) * ((H + sh - 1) / sh) * ((W + sw - 1) / sw);
                ATB_REQUIRE(ceil_div(C, 64) <= 65535, "C too large");
                launch_sgemm(p, max_class, C, sh * sw, s);
            } else {
                ConvGradX p{go, widx, dx, go_scale, w_zero, grad_x, N, O, static_cast<int>(K), g,
                            make_fastdiv(H * W), make_fastdiv(W), make_fastdiv(kh * kw), make_fastdiv(kw),
                            make_fastdiv(sh), make_fastdiv(sw), x_mask, x_scale};
                ATB_REQUIRE(ceil_div(C, 64) <= 65535, "C too large");
                launch_sgemm(p, Mx, C, 1, s);
            }
        }
        rc = check_launch("conv grad_x");
        if (rc != ATB_OK) return rc;
    }
    if (grad_w != nullptr && O * K > 0) {
        zero_kernel<<<grid_for(O * K, 256, 4096), 256, 0, s>>>(grad_w, O * K);
        rc = check_launch("zero_kernel");
        if (rc != ATB_OK) return rc;
        if (P > 0) {
            ATB_REQUIRE(go && x && dw, "null pointer");
            ATB_REQUIRE(ceil_div(K, 64) <= 65535, "K too large");
            const unsigned gz = split_factor(sgemm_tiles(O, K), P);
            if (lean && !simt_only) {
                rc = tc_conv_grad_w(go, x, x_dtype, dw, go_scale, grad_w, N, O, g, pad_index, exact_tables, s);
                if (rc != ATB_OK) return rc;
            } else if (lean) {
                const FastDiv dL = make_fastdiv(OH * OW), dOW = make_fastdiv(OW), dKK = make_fastdiv(kh * kw), dKW = make_fastdiv(kw);
                if (x_dtype == ATB_U8) {
                    ConvGradWLean<ATB_U8> p{go, x, dw, go_scale, grad_w, O, static_cast<int>(K), pad_index, P, g, dL, dOW, dKK, dKW};
                    launch_sgemm(p, O, K, gz, s);
                } else if (x_dtype == ATB_I8) {
                    ConvGradWLean<ATB_I8> p{go, x, dw, go_scale, grad_w, O, static_cast<int>(K), pad_index, P, g, dL, dOW, dKK, dKW};
                    launch_sgemm(p, O, K, gz, s);
                } else {
                    ConvGradWLean<ATB_F32> p{go, x, dw, go_scale, grad_w, O, static_cast<int>(K), pad_index, P, g, dL, dOW, dKK, dKW};
                    launch_sgemm(p, O, K, gz, s);
                }
            } else {
                ConvGradW p{go, x, x_dtype, dw, go_scale, grad_w, O, static_cast<int>(K), pad_index, P, g,
                            make_fastdiv(OH * OW), make_fastdiv(OW), make_fastdiv(kh * kw), make_fastdiv(kw)};
                launch_sgemm(p, O, K, gz, s);
            }
            rc = check_launch("conv grad_w");
        }
    }
    return rc;
}
