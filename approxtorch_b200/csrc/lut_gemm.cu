// LUT GEMM / approximate Conv2d forward for sm_100a.
//
//   acc[r, o] = sum_k lut[x_idx(r, k)][w_idx(o, k)]          r = pixel row (n, l), o = output channel
//
// A table lookup is not a dense contraction, so this kernel does not use the tensor cores; its
// roofline is the shared-memory load pipe (32 four-byte bank reads per clock per SM).  A plain
// gather from a 128 KB table in shared memory would spend ~3.4 bank wavefronts per 32 lookups on
// uniformly distributed operands, because 32 data-dependent addresses collide in the 32 banks.
// The kernel removes those collisions by construction and fetches four lookups per load:
//
//  * The whole transposed 16-bit table (128 KB) is resident in shared memory, stored so that a 32-bit word
//    of row w holds the entries {x = i, x = i + 128} and a lane's 16-byte load yields the four such pairs
//    (i = lane + 32 j) that the lane will write out.
//  * For every k-step the block STAGES the 64 table columns its 64 output channels need as 16 QUAD rows:
//    quad row p interleaves the columns of output channels p, p + 16, p + 32 and p + 48, its 8-byte entry x
//    being {T[w_p][x], T[w_p+16][x]} {T[w_p+32][x], T[w_p+48][x]}.  Building a quad row is four 16-byte
//    reads, 16 byte-permutes and eight conflict-free 8-byte writes per lane.
//  * The quad-row pitch is 2056 bytes (514 words, 2 mod 32).  An 8-byte shared load is served half a warp
//    at a time, and the 16 lanes of a half - one quad row each, the same activation value x (that of the
//    pixel row the half works on) - hit all 32 banks once: bank = (2 q + 2 x + {0, 1}) mod 32.  So a lookup
//    instruction costs one wavefront per 64 lookups and one instruction per 128.
//  * Each thread keeps 16 pixel rows x 4 output channels of exact integer accumulators in registers (a warp
//    32 rows x 64 channels), so staging one column (8 wavefronts) is amortised over `block_rows` (up to 512)
//    lookups.
//  * Entries are unsigned 16-bit (signed tables carry a +32768 bias removed in the epilogue).  A fetched
//    word v = lo + 65536*hi is accumulated as S0 += v and S1 += hi; the low channel's sum is
//    S0 - 65536*S1 (exact modulo 2^32; all sums stay below 2^31 because a block covers at most 32768 k-steps:
//    longer reductions are split along K and their partial sums added in 64 bits).
//
// Integer-valued tables (the int16 / uint16 images) accumulate exactly in int32.  Tables that are
// not 16-bit exact take the fp32 path: lookups go to the transposed fp32 table in global memory
// (L1/L2 resident) and are summed in fp32 in ascending k, as the reference does
// (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:278-281).
//
// The pixel operand is either a column matrix x[N,K,L] (L == 1: row-major A[M,K]) or the quantised
// image itself with the im2col gather done in the tile loader, so the conv never materialises the
// K/C-times larger column matrix (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:216-269
// is what it replaces).
#include "common.cuh"

namespace atb {

constexpr int kStagedCols = 64;                          // output channels per thread block
constexpr int kChunk = 16;                               // k-steps per operand tile
constexpr int kQuadRows = kStagedCols / 4;               // staged quad rows per k-step
constexpr int kQuadPitch = 2056;                         // bytes per quad row (256 x 4 x uint16 + 8 B skew)
constexpr int kStageBytes = kQuadRows * kQuadPitch;      // 32896
constexpr int kMaxBlockRows = 512;
constexpr int kTableBytes = 65536 * 2;
constexpr int kMaxBlockK = 32768;                        // k-steps one block may accumulate in its 32-bit sums
constexpr int kSmemStage = kTableBytes;
constexpr int kSmemX = kSmemStage + 2 * kStageBytes;
constexpr int kSmemW = kSmemX + 2 * kChunk * kMaxBlockRows;
constexpr int kSmemTotal = kSmemW + 2 * kChunk * kStagedCols;   // 215552 bytes

struct GemmArgs {
    const uint8_t* x;
    const uint8_t* w;
    const LutImage* img;
    float* y;
    int* scratch;          // split-K partials [S][srows][O] followed by row sums [S][srows]
    long long srow0, srows;   // pixel rows the split-K scratch covers: [srow0, srow0 + srows)
    int tile0;             // first row tile of this launch (added to blockIdx.x)
    // stream-K launches (sk_units > 0): the (tile, k-chunk) units, tile-major, are dealt out in equal contiguous
    // runs of sk_units, one run per block; a block works through the one to three tile segments of its run
    int sk_units, sk_col_tiles, block_rows;
    long long sk_total;    // fits 31 bits
    long long R;           // pixel rows
    int K, L, O;
    int wb_rows;           // pixel rows per weight matrix (0: one matrix for all rows)
    long long w_batch_stride;
    int tiles_per_batch;   // row tiles per weight batch (wb_rows != 0)
    int chunks_per_split, splits;
    int image_mode;        // 1: x is the quantised image, gather taps in the loader
    int x_xor;             // 0x80 when the image holds int8 values (idx = v + 128), else 0
    int pad_index;
    ConvGeom g;
    const float* alpha;
    const float* beta;
    const float* zero_x;
    const float* zero_w;
    const int* wsum;
};

// Epilogue arithmetic.  Integer tables: the sum, the zero-point terms and their combination are exact integers,
// converted to fp32 once (round to nearest even), then scaled and shifted.  One block's sum fits 32 bits (a block
// never covers more than 32768 k-steps); sums of split-K partials and the zero-point terms need 64.
__device__ __forceinline__ float scale_shift(float v, int o, const GemmArgs& a)
{
    if (a.alpha != nullptr) v = v * __ldg(a.alpha + o);
    if (a.beta != nullptr) v = v + __ldg(a.beta + o);
    return v;
}

__device__ __forceinline__ float finalize_output(long long total, long long xsum, int o, const GemmArgs& a)
{
    float v;
    if (a.zero_x != nullptr) {
        const long long zx = llrintf(__ldg(a.zero_x));
        const long long zw = llrintf(__ldg(a.zero_w + o));
        const long long ws = __ldg(a.wsum + o);
        v = __ll2float_rn(total - zw * xsum - zx * ws + static_cast<long long>(a.K) * zx * zw);
    } else {
        v = __ll2float_rn(total);
    }
    return scale_shift(v, o, a);
}

// Tables that are not 16-bit exact: the sum is already fp32; the zero-point terms (integers) are added in
// double so that they are not rounded before the one conversion back to fp32.
__device__ __forceinline__ float finalize_output(float total, long long xsum, int o, const GemmArgs& a)
{
    float v = total;
    if (a.zero_x != nullptr) {
        const long long zx = llrintf(__ldg(a.zero_x));
        const long long zw = llrintf(__ldg(a.zero_w + o));
        const long long ws = __ldg(a.wsum + o);
        v = static_cast<float>(static_cast<double>(total) +
                               static_cast<double>(-zw * xsum - zx * ws + static_cast<long long>(a.K) * zx * zw));
    }
    return scale_shift(v, o, a);
}

__device__ __forceinline__ long long output_offset(long long r, int o, const GemmArgs& a)
{
    const long long n = r / a.L;
    const long long l = r - n * a.L;
    return (n * a.O + o) * a.L + l;
}

// Position of output channel c (0..63 within the block) in a k-step's row of staged weight indices: the four
// channels of quad row p = c % 16 are adjacent.
__device__ __forceinline__ int w_slot(int c) { return ((c & (kQuadRows - 1)) << 2) + (c >> 4); }

// Quad row p interleaves the table columns of output channels p, p + 16, p + 32 and p + 48: its 8-byte entry x
// is {T[w_p][x], T[w_p+16][x]} (first word) and {T[w_p+32][x], T[w_p+48][x]} (second word).
struct QuadWords {
    uint32_t a[4], b[4], c[4], d[4];        // pairs {x = i, x = i + 128}, i = lane + 32 j, of the four columns
};

__device__ __forceinline__ void fetch_quad(const uint8_t* s_tab, const uint8_t* wstep, int p, int lane, QuadWords& v)
{
    const uint4* tab = reinterpret_cast<const uint4*>(s_tab);
    // the weight indices of a k-step are stored quad row by quad row (w_slot), so the four this quad row needs
    // arrive with one word load
    const uint32_t w4 = reinterpret_cast<const uint32_t*>(wstep)[p];
    const uint4 a4 = tab[(w4 & 0xffu) * 32u + lane];
    const uint4 b4 = tab[((w4 >> 8) & 0xffu) * 32u + lane];
    const uint4 c4 = tab[((w4 >> 16) & 0xffu) * 32u + lane];
    const uint4 d4 = tab[(w4 >> 24) * 32u + lane];
    v.a[0] = a4.x; v.a[1] = a4.y; v.a[2] = a4.z; v.a[3] = a4.w;
    v.b[0] = b4.x; v.b[1] = b4.y; v.b[2] = b4.z; v.b[3] = b4.w;
    v.c[0] = c4.x; v.c[1] = c4.y; v.c[2] = c4.z; v.c[3] = c4.w;
    v.d[0] = d4.x; v.d[1] = d4.y; v.d[2] = d4.z; v.d[3] = d4.w;
}

__device__ __forceinline__ void store_quad(uint8_t* stage, int p, int lane, const QuadWords& v)
{
    uint2* dst = reinterpret_cast<uint2*>(stage + p * kQuadPitch);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        dst[i] = make_uint2(__byte_perm(v.a[j], v.b[j], 0x5410), __byte_perm(v.c[j], v.d[j], 0x5410));        // x = i
        dst[i + 128] = make_uint2(__byte_perm(v.a[j], v.b[j], 0x7632), __byte_perm(v.c[j], v.d[j], 0x7632));  // x = i + 128
    }
}

// One k-step of staging: every warp builds its share of the 16 quad rows.
__device__ __forceinline__ void stage_quads(uint8_t* stage, const uint8_t* s_tab, const uint8_t* wstep,
                                            int warp, int lane, int nwarps)
{
    for (int p = warp; p < kQuadRows; p += nwarps) {
        QuadWords v;
        fetch_quad(s_tab, wstep, p, lane, v);
        store_quad(stage, p, lane, v);
    }
}

template <int TM>
__device__ __forceinline__ void load_x_words(const uint8_t* xrow, uint32_t (&xw)[TM / 4])
{
#pragma unroll
    for (int q = 0; q < TM / 16; ++q) {
        const uint4 v = *reinterpret_cast<const uint4*>(xrow + 16 * q);
        xw[4 * q] = v.x; xw[4 * q + 1] = v.y; xw[4 * q + 2] = v.z; xw[4 * q + 3] = v.w;
    }
}

// Lookups of one k-step.  Lane (h, q) = (lane / 16, lane % 16) works on 16 pixel rows (h * 16 + j of the
// warp's 32) and the four output channels of quad row q: per row ONE 8-byte load, then per word S0 += word
// and S1 += high half (a dot-product-accumulate that multiplies the halves by {0, 1}, or shift + add).
// An 8-byte shared load is served half a warp at a time, and the 16 lanes of a half (one quad row each, the
// same activation value x) hit all 32 banks once: bank = (2 q + 2 x + {0, 1}) mod 32.
template <bool DP2A>
__device__ __forceinline__ void lookup_step(const uint8_t* stage, const uint8_t* xrow16, int q, unsigned (&acc)[16][4])
{
    uint32_t xw[4];
    load_x_words<16>(xrow16, xw);
    const uint2* base = reinterpret_cast<const uint2*>(stage + q * kQuadPitch);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const uint2 v = base[__byte_perm(xw[j >> 2], 0, 0x4440 | (j & 3))];
        acc[j][0] += v.x;
        acc[j][2] += v.y;
        if constexpr (DP2A) {
            acc[j][1] = __dp2a_lo(v.x, 0x00000100u, acc[j][1]);
            acc[j][3] = __dp2a_lo(v.y, 0x00000100u, acc[j][3]);
        } else {
            acc[j][1] += v.x >> 16;
            acc[j][3] += v.y >> 16;
        }
    }
}

template <int TM>
__device__ __forceinline__ void lookup_step_f32(const float* tabT, const uint8_t* wstep, const uint8_t* xrow,
                                                int lane, float (&acc)[TM][2])
{
    uint32_t xw[TM / 4];
    load_x_words<TM>(xrow, xw);
    const float* c0 = tabT + (static_cast<uint32_t>(wstep[w_slot(lane)]) << 8);
    const float* c1 = tabT + (static_cast<uint32_t>(wstep[w_slot(lane + 32)]) << 8);
#pragma unroll
    for (int j = 0; j < TM; ++j) {
        const uint32_t xv = (xw[j >> 2] >> (8 * (j & 3))) & 0xffu;
        acc[j][0] += __ldg(c0 + xv);
        acc[j][1] += __ldg(c1 + xv);
    }
}

// Per-thread view of the pixel operand: thread t of the block loads row r0 + t of every k-step.
struct RowCursor {
    const uint8_t* base;   // column mode: &x[n, 0, l]; image mode: &x[n, 0, 0, 0]
    int ih0, iw0;          // image mode: top-left tap of the output pixel
};

__device__ __forceinline__ void load_chunk(const GemmArgs& a, const RowCursor& rc, const uint8_t* wcol,
                                           bool vec_x, bool vec_w, int k0, int kend, int tid, int pad,
                                           uint32_t (&xr)[4], uint32_t (&wr)[4], int bm)
{
    if (tid >= bm) {
        // threads beyond the tile's rows (16-rows-per-warp layout) load no pixel operand
    } else if (a.image_mode) {
        // Branch-free gather: every tap is loaded unconditionally (from the tap, or from the start of the sample
        // when the tap lies outside the image or past the last k) and the pad value is selected afterwards, so
        // that the 16 loads are independent and their latencies overlap.
        const int khw = a.g.KH * a.g.KW;
        int c = k0 / khw;
        const int rem = k0 - c * khw;
        int i = rem / a.g.KW;
        int j = rem - i * a.g.KW;
        uint32_t v[kChunk];
#pragma unroll
        for (int kk = 0; kk < kChunk; ++kk) {
            const int ih = rc.ih0 + i * a.g.DH;
            const int iw = rc.iw0 + j * a.g.DW;
            const bool inside = static_cast<unsigned>(ih) < static_cast<unsigned>(a.g.H) &&
                                static_cast<unsigned>(iw) < static_cast<unsigned>(a.g.W) && (k0 + kk < kend);
            const long long off = inside ? (static_cast<long long>(c) * a.g.H + ih) * a.g.W + iw : 0LL;
            const uint32_t b = static_cast<uint32_t>(__ldg(rc.base + off)) ^ static_cast<uint32_t>(a.x_xor);
            v[kk] = inside ? b : static_cast<uint32_t>(pad);
            const bool wrap_j = ++j == a.g.KW;
            j = wrap_j ? 0 : j;
            i += wrap_j ? 1 : 0;
            const bool wrap_i = i == a.g.KH;
            i = wrap_i ? 0 : i;
            c += wrap_i ? 1 : 0;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
            xr[q] = v[4 * q] | (v[4 * q + 1] << 8) | (v[4 * q + 2] << 16) | (v[4 * q + 3] << 24);
    } else if (vec_x) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(rc.base + k0));
        xr[0] = v.x; xr[1] = v.y; xr[2] = v.z; xr[3] = v.w;
    } else {
        xr[0] = xr[1] = xr[2] = xr[3] = 0u;
#pragma unroll
        for (int kk = 0; kk < kChunk; ++kk) {
            if (k0 + kk < kend) {
                const uint32_t v = __ldg(rc.base + static_cast<long long>(k0 + kk) * a.L);
                xr[kk >> 2] |= v << (8 * (kk & 3));
            }
        }
    }
    if (tid < kStagedCols) {
        if (vec_w) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(wcol + k0));
            wr[0] = v.x; wr[1] = v.y; wr[2] = v.z; wr[3] = v.w;
        } else {
            wr[0] = wr[1] = wr[2] = wr[3] = 0u;
#pragma unroll
            for (int kk = 0; kk < kChunk; ++kk) {
                if (k0 + kk < kend) {
                    const uint32_t v = __ldg(wcol + k0 + kk);
                    wr[kk >> 2] |= v << (8 * (kk & 3));
                }
            }
        }
    }
}

__device__ __forceinline__ void store_chunk(uint8_t* s_x, uint8_t* s_w, int buf, int tid,
                                            const uint32_t (&xr)[4], const uint32_t (&wr)[4], int bm)
{
    if (tid < bm) {
        uint8_t* xd = s_x + buf * kChunk * kMaxBlockRows + tid;
#pragma unroll
        for (int kk = 0; kk < kChunk; ++kk)
            xd[kk * kMaxBlockRows] = static_cast<uint8_t>(xr[kk >> 2] >> (8 * (kk & 3)));
    }
    if (tid < kStagedCols) {
        uint8_t* wd = s_w + buf * kChunk * kStagedCols + w_slot(tid);
#pragma unroll
        for (int kk = 0; kk < kChunk; ++kk)
            wd[kk * kStagedCols] = static_cast<uint8_t>(wr[kk >> 2] >> (8 * (kk & 3)));
    }
}

// Epilogue shared by both paths: `total(j, t)` yields the finished sum of this thread's row slot j, column slot t.
// QUAD = false (fp32 path): thread (warp, lane) holds pixel rows warp*32 + j (j = 0..31) of output channels
// lane and lane + 32.  QUAD = true (integer path): thread (warp, h, q) holds pixel rows warp*32 + h*16 + j
// (j = 0..15) of output channels q + 16 t (t = 0..3).  `xsum` is the operand sum of pixel row warp*32 + lane.
// Split-K partials and the L == 1 layout are written directly (lanes span consecutive channels, which is
// the fast axis there).  For L > 1 the fast axis of y[n, o, l] is the pixel, so each warp first turns its
// 32 x 64 tile around in shared memory (the table / stage area is free by now) and then stores 128
// contiguous bytes per channel.
template <bool QUAD, class Total, class Bits>
__device__ __forceinline__ void write_tile(const GemmArgs& a, uint8_t* smem, long long r0, long long r_end, int c0,
                                           int split, bool to_scratch,
                                           int warp, int lane, int xsum, Total total, Bits bits)
{
    constexpr int NJ = QUAD ? 16 : 32;               // row slots per thread
    constexpr int NT = QUAD ? 4 : 2;                 // column slots per thread
    const int row_base = QUAD ? (lane >> 4) * 16 : 0;        // first of this thread's rows within the warp's 32
    const int col_base = QUAD ? (lane & 15) : lane;          // first of this thread's columns within the 64
    constexpr int col_step = QUAD ? 16 : 32;
    const bool want_xsum = a.zero_x != nullptr;
    if (to_scratch || a.L == 1) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const long long r = r0 + warp * 32 + row_base + j;
            const int xs = __shfl_sync(0xffffffffu, xsum, row_base + j);
            if (r >= r_end) continue;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int o = c0 + col_base + col_step * t;
                if (o >= a.O) continue;
                if (to_scratch) a.scratch[(static_cast<long long>(split) * a.srows + (r - a.srow0)) * a.O + o] = bits(j, t);
                else a.y[output_offset(r, o, a)] = finalize_output(total(j, t), xs, o, a);
            }
            if (to_scratch && want_xsum && c0 == 0 && col_base == 0)
                a.scratch[static_cast<long long>(a.splits) * a.srows * a.O + static_cast<long long>(split) * a.srows + (r - a.srow0)] = xs;
        }
        return;
    }
    __syncthreads();                                   // every warp has left the main loop
    constexpr int kPitch = 33;                         // words per channel row of the turned tile
    float* tile = reinterpret_cast<float*>(smem) + warp * (kStagedCols * kPitch);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int xs = __shfl_sync(0xffffffffu, xsum, row_base + j);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int oc = col_base + col_step * t;
            tile[oc * kPitch + row_base + j] = (c0 + oc < a.O) ? finalize_output(total(j, t), xs, c0 + oc, a) : 0.0f;
        }
    }
    __syncwarp();
    const long long r = r0 + warp * 32 + lane;         // this lane's pixel row
    if (r < r_end) {
        const long long n = r / a.L;
        const long long l = r - n * a.L;
        float* dst = a.y + (n * a.O + c0) * a.L + l;
        const int ncols = min(kStagedCols, a.O - c0);
        for (int c = 0; c < ncols; ++c) dst[static_cast<long long>(c) * a.L] = tile[c * kPitch + lane];
    }
}

// 16-bit table classes: staged conflict-free lookups, exact integer accumulation.
// Software pipeline per k-step: issue the table reads for the NEXT step's quad rows, do this step's
// lookups (which hides the latency of those reads), permute and store the next step's quad rows into the
// other stage buffer, one barrier.
template <int NW, bool DP2A>
__device__ __forceinline__ void gemm_body_int(const GemmArgs& a, uint8_t* smem, const RowCursor& rc,
                                              const uint8_t* wcol, bool vec_x, bool vec_w, int pad, int bias,
                                              long long r0, long long r_end, int c0, int kbeg, int kend,
                                              int split, bool to_scratch, const volatile int* desc)
{
    constexpr int TM = 32;                       // pixel rows per warp
    constexpr bool kPipelined = NW >= kQuadRows; // one quad row per warp: keep the next step's table words in registers
    uint8_t* s_tab = smem;
    uint8_t* s_stage = smem + kSmemStage;
    uint8_t* s_x = smem + kSmemX;
    uint8_t* s_w = smem + kSmemW;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int q = lane & 15;                     // this lane's quad row
    const int h = lane >> 4;                     // which 16 of the warp's 32 pixel rows
    const int nch = (kend - kbeg + kChunk - 1) / kChunk;
    constexpr int bm = NW * TM;

    unsigned acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) { acc[j][0] = 0u; acc[j][1] = 0u; acc[j][2] = 0u; acc[j][3] = 0u; }
    int xsum = 0;
    const bool want_xsum = a.zero_x != nullptr;

    uint32_t xr[4], wr[4];
    if (nch > 0) {
        load_chunk(a, rc, wcol, vec_x, vec_w, kbeg, kend, tid, pad, xr, wr, bm);
        store_chunk(s_x, s_w, 0, tid, xr, wr, bm);
    }
    __syncthreads();          // table image and first operand tile are in shared memory
    if (nch > 0) {
        stage_quads(s_stage, s_tab, s_w, warp, lane, NW);
        __syncthreads();
    }

    int step = 0;
    for (int ci = 0; ci < nch; ++ci) {
        const int k0 = kbeg + ci * kChunk;
        const int kc = min(kChunk, kend - k0);
        const int cur = ci & 1;
        const bool has_next = ci + 1 < nch;
        if (has_next) load_chunk(a, rc, wcol, vec_x, vec_w, k0 + kChunk, kend, tid, pad, xr, wr, bm);
        for (int kk = 0; kk < kc; ++kk, ++step) {
            if (has_next && kk == 4) store_chunk(s_x, s_w, cur ^ 1, tid, xr, wr, bm);
            const uint8_t* xrow = s_x + (cur * kChunk + kk) * kMaxBlockRows + warp * TM;
            const uint8_t* wstep = s_w + (cur * kChunk + kk) * kStagedCols;
            const uint8_t* wnext = nullptr;
            if (kk + 1 < kc) wnext = wstep + kStagedCols;
            else if (has_next) wnext = s_w + ((cur ^ 1) * kChunk) * kStagedCols;
            uint8_t* stage_next = s_stage + ((step + 1) & 1) * kStageBytes;
            const uint8_t* stage_cur = s_stage + (step & 1) * kStageBytes;
            if (want_xsum) xsum += static_cast<int>(xrow[lane]);

            if constexpr (kPipelined) {
                QuadWords v;
                if (wnext != nullptr && warp < kQuadRows) fetch_quad(s_tab, wnext, warp, lane, v);
                lookup_step<DP2A>(stage_cur, xrow + h * 16, q, acc);
                if (wnext != nullptr && warp < kQuadRows) store_quad(stage_next, warp, lane, v);
            } else {
                if (wnext != nullptr) stage_quads(stage_next, s_tab, wnext, warp, lane, NW);
                lookup_step<DP2A>(stage_cur, xrow + h * 16, q, acc);
            }
            __syncthreads();
        }
    }
    const long long remove = static_cast<long long>(bias) * (kend - kbeg);     // +32768 per looked-up entry of a signed table
    // per word: acc[j][2u] holds sum(lo) + 65536 * sum(hi) modulo 2^32, acc[j][2u + 1] holds sum(hi)
    auto total = [&](int j, int t) -> long long {
        const int u = (t >> 1) * 2;
        const unsigned v = (t & 1) == 0 ? acc[j][u] - (acc[j][u + 1] << 16) : acc[j][u + 1];
        return static_cast<long long>(v) - remove;
    };
    if (desc != nullptr) {
        // stream-K: the tile coordinates were not kept in registers across the main loop; read them back
        r0 = static_cast<long long>(desc[0]) * bm;
        c0 = desc[1];
        split = desc[4];
    }
    write_tile<true>(a, smem, r0, r_end, c0, split, to_scratch, warp, lane, xsum,
                     [&](int j, int t) { return total(j, t); },
                     [&](int j, int t) { return static_cast<int>(total(j, t)); });
}

// Tables that are not 16-bit exact: lookups from the transposed fp32 table in global memory,
// fp32 accumulation in ascending k.
template <int TM>
__device__ __forceinline__ void gemm_body_f32(const GemmArgs& a, uint8_t* smem, const RowCursor& rc,
                                              const uint8_t* wcol, bool vec_x, bool vec_w, int pad,
                                              long long r0, long long r_end, int c0, int kbeg, int kend,
                                              int split, bool to_scratch, const volatile int* desc)
{
    uint8_t* s_x = smem + kSmemX;
    uint8_t* s_w = smem + kSmemW;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int nch = (kend - kbeg + kChunk - 1) / kChunk;

    const int bm = (blockDim.x >> 5) * TM;
    float acc[TM][2];
#pragma unroll
    for (int j = 0; j < TM; ++j) { acc[j][0] = 0.0f; acc[j][1] = 0.0f; }
    int xsum = 0;
    const bool want_xsum = a.zero_x != nullptr;

    uint32_t xr[4], wr[4];
    if (nch > 0) {
        load_chunk(a, rc, wcol, vec_x, vec_w, kbeg, kend, tid, pad, xr, wr, bm);
        store_chunk(s_x, s_w, 0, tid, xr, wr, bm);
    }
    __syncthreads();
    for (int ci = 0; ci < nch; ++ci) {
        const int k0 = kbeg + ci * kChunk;
        const int kc = min(kChunk, kend - k0);
        const int cur = ci & 1;
        const bool has_next = ci + 1 < nch;
        if (has_next) load_chunk(a, rc, wcol, vec_x, vec_w, k0 + kChunk, kend, tid, pad, xr, wr, bm);
        for (int kk = 0; kk < kc; ++kk) {
            if (has_next && kk == 4) store_chunk(s_x, s_w, cur ^ 1, tid, xr, wr, bm);
            const uint8_t* xrow = s_x + (cur * kChunk + kk) * kMaxBlockRows + warp * TM;
            const uint8_t* wstep = s_w + (cur * kChunk + kk) * kStagedCols;
            if (want_xsum && lane < TM) xsum += static_cast<int>(xrow[lane]);
            lookup_step_f32<TM>(a.img->tabT32, wstep, xrow, lane, acc);
        }
        __syncthreads();
    }
    if (desc != nullptr) {
        r0 = static_cast<long long>(desc[0]) * bm;
        c0 = desc[1];
        split = desc[4];
    }
    write_tile<false>(a, smem, r0, r_end, c0, split, to_scratch, warp, lane, xsum,
               [&](int j, int t) { return acc[j][t]; },
               [&](int j, int t) { return __float_as_int(acc[j][t]); });
}

// One tile segment: rows of row tile `row_tile`, the 64 output channels from c0, k-chunks [ch_beg, ch_end).
// The result goes to y (to_scratch false) or, as a partial sum, to slot `split` of the scratch.
template <int NW, bool DP2A>
__device__ __forceinline__ void run_segment(const GemmArgs& a, uint8_t* smem, int cls, int row_tile, int c0,
                                            int ch_beg, int ch_end, int split, bool to_scratch,
                                            const volatile int* desc = nullptr)
{
    constexpr int TM = 32;
    const int tid = threadIdx.x;
    constexpr int bm = NW * TM;

    long long r0, r_end;
    long long wbatch = 0;
    if (a.wb_rows > 0) {
        wbatch = row_tile / a.tiles_per_batch;
        const int t = row_tile - static_cast<int>(wbatch) * a.tiles_per_batch;
        r0 = wbatch * a.wb_rows + static_cast<long long>(t) * bm;
        r_end = min(a.R, (wbatch + 1) * a.wb_rows);
    } else {
        r0 = static_cast<long long>(row_tile) * bm;
        r_end = a.R;
    }
    const int kbeg = ch_beg * kChunk;
    const int kend = min(a.K, ch_end * kChunk);

    // this thread's pixel row for the tile loads (clamped: rows past the end are never stored)
    const long long r = min(r0 + min(tid, bm - 1), r_end - 1);
    RowCursor rc;
    bool vec_x = false;
    if (a.image_mode) {
        const long long hw = static_cast<long long>(a.g.OH) * a.g.OW;
        const long long n = r / hw;
        const int rem = static_cast<int>(r - n * hw);
        const int oh = rem / a.g.OW;
        const int ow = rem - oh * a.g.OW;
        rc.base = a.x + n * a.g.C * a.g.H * a.g.W;
        rc.ih0 = oh * a.g.SH - a.g.PH;
        rc.iw0 = ow * a.g.SW - a.g.PW;
    } else {
        const long long n = r / a.L;
        const long long l = r - n * a.L;
        rc.base = a.x + n * a.K * a.L + l;
        rc.ih0 = rc.iw0 = 0;
        vec_x = (a.L == 1) && (a.K % kChunk == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
    }
    const int ocol = min(c0 + tid, a.O - 1);
    const uint8_t* wcol = a.w + wbatch * a.w_batch_stride + static_cast<long long>(ocol) * a.K;
    const bool vec_w = (a.K % kChunk == 0) && ((reinterpret_cast<uintptr_t>(a.w) & 15) == 0) &&
                       ((a.w_batch_stride & 15) == 0);
    // pad_index < 0: taps outside the image take the activation zero point (an integer-valued device scalar)
    const int pad = a.pad_index >= 0 ? a.pad_index : min(255, max(0, static_cast<int>(llrintf(__ldg(a.zero_x)))));
    if (cls != LUT_F32)
        gemm_body_int<NW, DP2A>(a, smem, rc, wcol, vec_x, vec_w, pad, cls == LUT_I16 ? 32768 : 0, r0, r_end, c0, kbeg, kend,
                                split, to_scratch, desc);
    else
        gemm_body_f32<TM>(a, smem, rc, wcol, vec_x, vec_w, pad, r0, r_end, c0, kbeg, kend, split, to_scratch, desc);
}

// NW warps per block, 32 pixel rows per warp (one thread per row loads the operand tiles, 64 accumulators
// per thread).  DP2A selects how the high half of a fetched word is accumulated.
// SK: the block works through a run of tile segments (stream-K) instead of one tile or tile split.
template <int NW, bool DP2A, bool SK>
__global__ void __launch_bounds__(NW * 32, 1) lut_gemm_kernel(const GemmArgs a)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x;
    const int cls = lut_class_of(a.img);
    if (cls != LUT_F32) {
        // The image holds the table as the lookups want it (signed entries biased by +32768, so every lookup is an
        // unsigned 16-bit load): asynchronous 16-byte copies straight into shared memory, all in flight at once.
        const char* src = reinterpret_cast<const char*>(a.img->tabTP16);
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
        for (int i = tid; i < kTableBytes / 16; i += blockDim.x)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + 16 * i) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");     // visible to the block after the next barrier
    }
    const int nchunks = (a.K + kChunk - 1) / kChunk;
    if constexpr (!SK) {
        const int ch_beg = blockIdx.z * a.chunks_per_split;
        run_segment<NW, DP2A>(a, smem, cls, a.tile0 + static_cast<int>(blockIdx.x), blockIdx.y * kStagedCols,
                              ch_beg, min(nchunks, ch_beg + a.chunks_per_split), blockIdx.z, a.splits > 1);
    } else {
        // This block's run of (tile, k-chunk) units; the table image stays in shared memory throughout.  The main
        // loop has no register to spare, so the description of the current segment lives in shared memory: thread
        // 0 writes it, everybody reads it for the prologue, and the epilogue and the loop read it back.
        __shared__ int s_desc[8];        // row tile, first column, first chunk, end chunk, segment number, next unit
        int u = static_cast<int>(blockIdx.x) * a.sk_units;
        while (true) {
            if (tid == 0) {
                const int u_end = static_cast<int>(min(a.sk_total, static_cast<long long>(blockIdx.x + 1) * a.sk_units));
                const int tile = u / nchunks;
                const int ch_beg = u - tile * nchunks;
                const int ch_end = min(nchunks, ch_beg + (u_end - u));
                const int row_tile = tile / a.sk_col_tiles;
                s_desc[0] = row_tile;
                s_desc[1] = (tile - row_tile * a.sk_col_tiles) * kStagedCols;
                s_desc[2] = ch_beg;
                s_desc[3] = ch_end;
                // segments of one tile are numbered by the blocks that hold them, in k order
                s_desc[4] = u / a.sk_units - (tile * nchunks) / a.sk_units;
                s_desc[5] = u + (ch_end - ch_beg);
                s_desc[6] = u_end;
            }
            __syncthreads();
            run_segment<NW, DP2A>(a, smem, cls, s_desc[0], s_desc[1], s_desc[2], s_desc[3], s_desc[4], true,
                                  const_cast<const volatile int*>(s_desc));
            const volatile int* d = s_desc;
            u = d[5];
            const int u_end = d[6];
            __syncthreads();             // everybody has read the description before thread 0 rewrites it
            if (u >= u_end) break;
        }
    }
}

// Split-K: y = finalize(sum_s partial[s]) in ascending split order, over the rows the scratch covers.
__global__ void lut_gemm_reduce_kernel(const GemmArgs a)
{
    const long long total = a.srows * a.O;
    const int cls = lut_class_of(a.img);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const int nchunks = (a.K + kChunk - 1) / kChunk;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long rs = i / a.O;
        const int o = static_cast<int>(i - rs * a.O);
        // number of partial sums of this element, and of its row's operand sum (held by the first column tile)
        int ns = a.splits, nx = a.splits;
        if (a.sk_units > 0) {
            const long long t0 = (rs / a.block_rows) * a.sk_col_tiles;                   // first tile of the row tile
            const long long t1 = t0 + o / kStagedCols;
            nx = static_cast<int>((t0 * nchunks + nchunks - 1) / a.sk_units - (t0 * nchunks) / a.sk_units) + 1;
            ns = static_cast<int>((t1 * nchunks + nchunks - 1) / a.sk_units - (t1 * nchunks) / a.sk_units) + 1;
        }
        long long xs = 0;
        if (a.zero_x != nullptr)
            for (int s = 0; s < nx; ++s) xs += a.scratch[a.splits * total + static_cast<long long>(s) * a.srows + rs];
        float v;
        if (cls == LUT_F32) {
            float f = 0.0f;
            for (int s = 0; s < ns; ++s) f += __int_as_float(a.scratch[static_cast<long long>(s) * total + i]);
            v = finalize_output(f, xs, o, a);
        } else {
            long long t = 0;
            for (int s = 0; s < ns; ++s) t += a.scratch[static_cast<long long>(s) * total + i];
            v = finalize_output(t, xs, o, a);
        }
        a.y[output_offset(a.srow0 + rs, o, a)] = v;
    }
}

// K == 0: exact zeros through the same epilogue (approxtorch/backend/csrc/claude/gemm.cu:30-32)
__global__ void lut_gemm_empty_k_kernel(const GemmArgs a)
{
    const long long total = a.R * a.O;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / a.O;
        const int o = static_cast<int>(i - r * a.O);
        a.y[output_offset(r, o, a)] = finalize_output(0LL, 0, o, a);
    }
}

// First pixel row of row tile t.
static long long tile_first_row(long long t, int bm, int wb_rows, int tiles_per_batch)
{
    if (wb_rows > 0) return (t / tiles_per_batch) * wb_rows + (t % tiles_per_batch) * static_cast<long long>(bm);
    return t * bm;
}

// Modelled duration of `blocks` equal thread blocks of `ksteps` k-steps each, in k-step units: whole waves
// of `sms` blocks, each paying a fixed prologue (table image into shared memory, first operand tile) and
// epilogue worth about a dozen k-steps.
static double wave_cost(long long blocks, int ksteps, int sms)
{
    constexpr double kFixed = 12.0;
    return static_cast<double>((blocks + sms - 1) / sms) * (ksteps + kFixed);
}

static int make_plan(long long R, int K, int O, int wb_rows, int cfg, atb_gemm_plan* p,
                     int* tiles_per_batch, long long* row_tiles)
{
    ATB_REQUIRE(p != nullptr, "plan is null");
    ATB_REQUIRE(R >= 0 && K >= 0 && O >= 0 && wb_rows >= 0, "negative dimension");
    const int sms = sm_count();
    const long long span = wb_rows > 0 ? wb_rows : R;
    int bm = 0, splits = 0;
    bool allow_tail = true;
    if (cfg >= 0) { bm = cfg & 0xffff; splits = (cfg >> 16) & 0xff; allow_tail = ((cfg >> 25) & 1) == 0; }
    if (bm != 0) {
        ATB_REQUIRE(bm == 64 || bm == 128 || bm == 256 || bm == 512, "cfg: block rows must be 64, 128, 256 or 512");
    } else {
        // 32 staged pair rows divide evenly over 2, 4, 8 or 16 warps; a warp covers 32 pixel rows
        bm = 64;
        while (bm < kMaxBlockRows && bm < span) bm *= 2;
    }
    const int tpb = wb_rows > 0 ? ceil_div(wb_rows, bm) : 0;
    const long long rt = wb_rows > 0 ? (R / (wb_rows > 0 ? wb_rows : 1)) * tpb : (R + bm - 1) / bm;
    const int ct = ceil_div(O > 0 ? O : 1, kStagedCols);
    const long long tiles = rt * ct;
    const int nchunks = K > 0 ? ceil_div(K, kChunk) : 1;
    long long tail_rt = 0;
    int sk_units = 0;
    bool allow_sk = wb_rows == 0 && (cfg < 0 || (((cfg >> 26) & 1) == 0 && splits == 0));
    // A block's 32-bit accumulators hold at most kMaxBlockK looked-up 16-bit entries, so longer reductions are
    // always split along K (the reduction pass adds the partial sums in 64 bits).
    const int min_splits = ceil_div(nchunks, kMaxBlockK / kChunk);
    if (min_splits > 1) { allow_tail = false; allow_sk = false; }
    if (splits == 0) {
        splits = 1;
        double classic = wave_cost(tiles, K, sms);      // modelled cost of the plan chosen so far
        // (1) Grids of more than one wave whose last wave is ragged: the whole waves run unsplit, and only
        // the trailing row tiles are split along K so that they fill one more (shorter) wave.  Their partial
        // sums are the only ones that go through scratch.
        if (allow_tail && tiles > sms && tiles % sms != 0 && nchunks > 1) {
            const long long full = tiles / sms;
            const long long main_rt = (full * sms) / ct;
            const long long t_rt = rt - main_rt;
            if (main_rt > 0 && t_rt > 0) {
                const double base = wave_cost(tiles, K, sms);
                double best = base;
                int best_s = 1;
                for (int s = 2; s <= 16 && s <= nchunks; ++s) {
                    const int cps = ceil_div(nchunks, s);
                    const int s_eff = ceil_div(nchunks, cps);
                    const double cost = wave_cost(main_rt * ct, K, sms) + wave_cost(t_rt * ct * s_eff, cps * kChunk, sms) + 6.0;
                    if (cost < best - 1e-9) { best = cost; best_s = s; }
                }
                if (best_s > 1 && best <= 0.95 * base) { splits = best_s; tail_rt = t_rt; classic = best; }
            }
        }
        // (2) Otherwise split-K over all tiles, by the same model: S_eff equal parts of ceil(chunks / S) chunks
        // each, whole waves of `sms` blocks, a fixed cost per block and a reduction pass.  Grids that already
        // fill the GPU only split for a modelled gain of 10 % or more (the partial sums need S times the output
        // in scratch).
        if (tail_rt == 0 && tiles > 0 && tiles < 4LL * sms && nchunks > 1) {
            const double base = wave_cost(tiles, K, sms);
            double best = base;
            int best_s = 1;
            for (int s = 2; s <= 16 && s <= nchunks; ++s) {
                const int cps = ceil_div(nchunks, s);
                const int s_eff = ceil_div(nchunks, cps);
                if (s_eff != s) continue;                       // same launch as a smaller s
                // partial sums: S_eff * R * O int32 written and read back, ~2e-6 k-step times per element
                const double traffic = 2.1e-6 * s_eff * static_cast<double>(R) * O;
                const double cost = wave_cost(tiles * s_eff, cps * kChunk, sms) + 6.0 + traffic;
                if (cost < best - 1e-9) { best = cost; best_s = s; }
            }
            if (best_s > 1 && (tiles < sms ? best <= 0.97 * base : best <= 0.9 * base)) { splits = best_s; classic = best; }
        }
        // (3) Stream-K for grids of a few waves at most: the (tile, k-chunk) units, tile-major, are dealt out in
        // equal contiguous runs, one per SM, so every SM gets the same number of k-steps whatever the tile count.
        // A block loads the table once and works through the one to three tile segments of its run; every
        // segment's partial sums go through scratch and the reduction pass finishes all outputs.
        if (allow_sk && tiles > 0 && (tiles < 4LL * sms || (cfg >= 0 && ((cfg >> 27) & 1))) && nchunks > 1) {
            const long long total = tiles * nchunks;
            const long long ctas = total < sms ? total : sms;
            const long long units = (total + ctas - 1) / ctas;
            const double segs = static_cast<double>((units + nchunks - 1) / nchunks + 1);
            const double traffic = 2.1e-6 * 2.5 * static_cast<double>(R) * O;
            const double cost = static_cast<double>(units) * kChunk + 8.0 * segs + 6.0 + traffic;
            const bool forced = cfg >= 0 && ((cfg >> 27) & 1);
            if ((forced || cost <= 0.95 * classic) && total < 2147483647LL / 2) {
                sk_units = static_cast<int>(units);
                tail_rt = 0;
                splits = static_cast<int>((nchunks + units - 2) / units + 1);     // most segments any tile can have
            }
        }
    }
    if (splits < min_splits) splits = min_splits;
    if (sk_units == 0) {
        if (splits > nchunks) splits = nchunks;
        const int cps = ceil_div(nchunks, splits);
        splits = ceil_div(nchunks, cps);
        if (splits == 1) tail_rt = 0;
    }
    const long long srow0 = tail_rt > 0 ? tile_first_row(rt - tail_rt, bm, wb_rows, tpb) : 0;
    p->block_rows = bm;
    p->splits = splits;
    p->scratch_bytes = (splits > 1 || sk_units > 0)
                           ? static_cast<size_t>(splits) * static_cast<size_t>(R - srow0) * (static_cast<size_t>(O) + 1) * 4u : 0u;
    p->tail_row_tiles = static_cast<int>(tail_rt);
    p->stream_k_units = sk_units;
    if (tiles_per_batch) *tiles_per_batch = tpb;
    if (row_tiles) *row_tiles = rt;
    return ATB_OK;
}

template <int NW, bool DP2A, bool SK>
static int launch_one(dim3 grid, const GemmArgs& a, cudaStream_t stream)
{
    // the opt-in shared-memory size is an attribute of the function on ONE device: set it once per device
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return ATB_ERR_CUDA;
    }
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(lut_gemm_kernel<NW, DP2A, SK>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        attr_set[dev] = true;
    }
    lut_gemm_kernel<NW, DP2A, SK><<<grid, NW * 32, kSmemTotal, stream>>>(a);
    return ATB_OK;
}

// stream-K launches always accumulate with the dot-product instruction
static int launch_variant(int nwarps, bool dp2a, bool sk, dim3 grid, const GemmArgs& a, cudaStream_t stream)
{
    switch (nwarps) {
        case 16: return sk ? launch_one<16, true, true>(grid, a, stream)
                           : dp2a ? launch_one<16, true, false>(grid, a, stream) : launch_one<16, false, false>(grid, a, stream);
        case 8: return sk ? launch_one<8, true, true>(grid, a, stream)
                          : dp2a ? launch_one<8, true, false>(grid, a, stream) : launch_one<8, false, false>(grid, a, stream);
        case 4: return sk ? launch_one<4, true, true>(grid, a, stream)
                          : dp2a ? launch_one<4, true, false>(grid, a, stream) : launch_one<4, false, false>(grid, a, stream);
        case 2: return sk ? launch_one<2, true, true>(grid, a, stream)
                          : dp2a ? launch_one<2, true, false>(grid, a, stream) : launch_one<2, false, false>(grid, a, stream);
        default: set_error("block rows must be 64, 128, 256 or 512"); return ATB_ERR_INVALID;
    }
}

static int launch_gemm(GemmArgs a, int cfg, void* scratch, size_t scratch_bytes, cudaStream_t stream)
{
    if (a.R == 0 || a.O == 0) return ATB_OK;
    ATB_REQUIRE(a.wb_rows == 0 || a.R % a.wb_rows == 0, "rows must be a multiple of wb_rows");
    if (a.K == 0) {
        lut_gemm_empty_k_kernel<<<grid_for(a.R * a.O, 256, 4096), 256, 0, stream>>>(a);
        return check_launch("lut_gemm_empty_k_kernel");
    }
    atb_gemm_plan plan;
    int tpb = 0;
    long long row_tiles = 0;
    int rc = make_plan(a.R, a.K, a.O, a.wb_rows, cfg, &plan, &tpb, &row_tiles);
    if (rc != ATB_OK) return rc;
    ATB_REQUIRE(row_tiles <= 2147483647LL, "too many row tiles");
    const int col_tiles = ceil_div(a.O, kStagedCols);
    ATB_REQUIRE(col_tiles <= 65535, "too many output channels");
    ATB_REQUIRE(plan.splits <= 65535, "K too large");
    if (plan.scratch_bytes > 0) {
        if (scratch == nullptr || scratch_bytes < plan.scratch_bytes) {
            set_error("split-K needs %zu bytes of scratch, got %zu", plan.scratch_bytes, scratch_bytes);
            return ATB_ERR_SCRATCH;
        }
    }
    a.scratch = static_cast<int*>(scratch);
    a.tiles_per_batch = tpb;
    const bool shift_add = cfg >= 0 && ((cfg >> 24) & 1);      // cfg bit 24: accumulate high halves with shift + add
    const int nchunks = ceil_div(a.K, kChunk);
    a.block_rows = plan.block_rows;
    if (plan.stream_k_units > 0) {
        a.tile0 = 0; a.splits = plan.splits; a.chunks_per_split = nchunks; a.srow0 = 0; a.srows = a.R;
        a.sk_units = plan.stream_k_units; a.sk_col_tiles = col_tiles;
        a.sk_total = row_tiles * col_tiles * nchunks;
        dim3 grid(static_cast<unsigned>((a.sk_total + a.sk_units - 1) / a.sk_units), 1u, 1u);
        rc = launch_variant(plan.block_rows / 32, true, true, grid, a, stream);
        if (rc != ATB_OK) return rc;
        rc = check_launch("lut_gemm_kernel");
        if (rc != ATB_OK) return rc;
        lut_gemm_reduce_kernel<<<grid_for(a.srows * a.O, 256, 8 * sm_count()), 256, 0, stream>>>(a);
        return check_launch("lut_gemm_reduce_kernel");
    }
    const long long tail_rt = plan.tail_row_tiles;
    const long long main_rt = row_tiles - tail_rt;
    if (tail_rt > 0) {
        // whole waves, unsplit
        a.tile0 = 0; a.splits = 1; a.chunks_per_split = nchunks; a.srow0 = 0; a.srows = a.R;
        dim3 grid(static_cast<unsigned>(main_rt), static_cast<unsigned>(col_tiles), 1u);
        rc = launch_variant(plan.block_rows / 32, !shift_add, false, grid, a, stream);
        if (rc != ATB_OK) return rc;
        rc = check_launch("lut_gemm_kernel");
        if (rc != ATB_OK) return rc;
    }
    // the split-K part: every tile, or only the trailing row tiles
    a.tile0 = static_cast<int>(main_rt) * (tail_rt > 0 ? 1 : 0);
    a.splits = plan.splits;
    a.chunks_per_split = ceil_div(nchunks, plan.splits);
    a.srow0 = tail_rt > 0 ? tile_first_row(main_rt, plan.block_rows, a.wb_rows, tpb) : 0;
    a.srows = a.R - a.srow0;
    dim3 grid(static_cast<unsigned>(tail_rt > 0 ? tail_rt : row_tiles), static_cast<unsigned>(col_tiles),
              static_cast<unsigned>(plan.splits));
    rc = launch_variant(plan.block_rows / 32, !shift_add, false, grid, a, stream);
    if (rc != ATB_OK) return rc;
    rc = check_launch("lut_gemm_kernel");
    if (rc != ATB_OK) return rc;
    if (plan.splits > 1) {
        lut_gemm_reduce_kernel<<<grid_for(a.srows * a.O, 256, 8 * sm_count()), 256, 0, stream>>>(a);
        rc = check_launch("lut_gemm_reduce_kernel");
    }
    return rc;
}

}  // namespace atb

using namespace atb;

extern "C" int atb_lut_gemm_plan(long long R, int K, int O, int wb_rows, int cfg, atb_gemm_plan* plan)
{
    return make_plan(R, K, O, wb_rows, cfg, plan, nullptr, nullptr);
}

static int check_epilogue(const float* zero_x, const float* zero_w, const int* wsum)
{
    if (zero_x != nullptr) ATB_REQUIRE(zero_w != nullptr && wsum != nullptr, "zero_x needs zero_w and wsum");
    return ATB_OK;
}

extern "C" int atb_lut_bgemm_fwd(const uint8_t* x, const uint8_t* w, const void* lut_image, float* y,
                                 int N, int K, int L, int O, int wb_rows, long long w_batch_stride,
                                 const float* alpha, const float* beta, const float* zero_x,
                                 const float* zero_w, const int* wsum,
                                 int cfg, void* scratch, size_t scratch_bytes, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    ATB_REQUIRE(lut_image != nullptr, "lut_image is null");
    if (static_cast<long long>(N) * L == 0 || O == 0) return ATB_OK;
    ATB_REQUIRE(y != nullptr && (K == 0 || (x != nullptr && w != nullptr)), "null operand");
    int rc = check_epilogue(zero_x, zero_w, wsum);
    if (rc != ATB_OK) return rc;
    GemmArgs a{};
    a.x = x; a.w = w; a.img = static_cast<const LutImage*>(lut_image); a.y = y;
    a.R = static_cast<long long>(N) * L; a.K = K; a.L = L; a.O = O;
    a.wb_rows = wb_rows; a.w_batch_stride = w_batch_stride;
    a.image_mode = 0; a.x_xor = 0; a.pad_index = 0;
    a.alpha = alpha; a.beta = beta; a.zero_x = zero_x; a.zero_w = zero_w; a.wsum = wsum;
    return launch_gemm(a, cfg, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

// ---- entry point for callers that cannot allocate device memory ------------------------------------
// Split-K partial sums normally go to a caller-supplied scratch buffer.  Some hosts of this library
// cannot provide one: code running inside a CUDA-graph capture or under a memory pool that forbids new
// allocations, and bindings from runtimes whose tensors cannot be created from inside an operator call.
// For them the library carries its own fixed scratch area in device global memory.  It exists once per
// GPU that loads the library and is held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[ATB_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void** out)
{
    // The symbol name is only a host-side handle: the device address has to be asked for, once per
    // device, while that device is current.  Threads that race here all store the same value.
    static void* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return ATB_ERR_CUDA;
    }
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
            return ATB_ERR_CUDA;
        }
        cached[dev] = p;
    }
    *out = cached[dev];
    return ATB_OK;
}

// Also performs the per-device address lookup for the current device, so that a host can get it out of the way
// before a stream capture without running a GEMM (a failure here is reported again by the GEMM call).
extern "C" size_t atb_static_scratch_bytes(void)
{
    void* unused = nullptr;
    (void)static_scratch_address(&unused);
    return ATB_STATIC_SCRATCH_BYTES;
}

extern "C" int atb_lut_bgemm_fwd_noalloc(const uint8_t* x, const uint8_t* w, const void* lut_image, float* y,
                                         int N, int K, int L, int O, int wb_rows, long long w_batch_stride,
                                         const float* alpha, const float* beta, const float* zero_x,
                                         const float* zero_w, const int* wsum, int cfg, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    atb_gemm_plan plan;
    int rc = make_plan(static_cast<long long>(N) * L, K, O, wb_rows, cfg, &plan, nullptr, nullptr);
    if (rc != ATB_OK) return rc;
    if (plan.scratch_bytes > ATB_STATIC_SCRATCH_BYTES) {
        set_error("this shape needs %zu bytes of split-K scratch but the built-in area holds %zu; "
                  "use atb_lut_bgemm_fwd with a caller buffer, or force fewer splits through cfg",
                  plan.scratch_bytes, static_cast<size_t>(ATB_STATIC_SCRATCH_BYTES));
        return ATB_ERR_SCRATCH;
    }
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != ATB_OK) return rc;
    return atb_lut_bgemm_fwd(x, w, lut_image, y, N, K, L, O, wb_rows, w_batch_stride, alpha, beta, zero_x, zero_w,
                             wsum, cfg, scratch, ATB_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int atb_lut_conv2d_fwd(const void* x, int dtype, const uint8_t* w, const void* lut_image, float* y,
                                  int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw,
                                  int ph, int pw, int dh, int dw, int pad_index,
                                  const float* alpha, const float* beta, const float* zero_x,
                                  const float* zero_w, const int* wsum,
                                  int cfg, void* scratch, size_t scratch_bytes, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0 && O >= 0, "negative dimension");
    ATB_REQUIRE(dtype == ATB_I8 || dtype == ATB_U8, "image must be int8 values or uint8 indices");
    ATB_REQUIRE(pad_index >= -1 && pad_index <= 255, "pad_index out of range");
    ATB_REQUIRE(pad_index >= 0 || zero_x != nullptr, "pad_index -1 takes the pad value from zero_x, which is null");
    ATB_REQUIRE(lut_image != nullptr, "lut_image is null");
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw, &OH, &OW), "conv geometry yields empty output");
    if (N == 0 || O == 0) return ATB_OK;
    const long long K = static_cast<long long>(C) * kh * kw;
    ATB_REQUIRE(K <= 2147483647LL - kChunk, "C*kh*kw too large");
    ATB_REQUIRE(y != nullptr && (K == 0 || (x != nullptr && w != nullptr)), "null operand");
    int rc = check_epilogue(zero_x, zero_w, wsum);
    if (rc != ATB_OK) return rc;
    GemmArgs a{};
    a.x = static_cast<const uint8_t*>(x); a.w = w; a.img = static_cast<const LutImage*>(lut_image); a.y = y;
    a.L = OH * OW; a.R = static_cast<long long>(N) * a.L; a.K = static_cast<int>(K); a.O = O;
    a.wb_rows = 0; a.w_batch_stride = 0;
    a.image_mode = 1; a.x_xor = (dtype == ATB_I8) ? 0x80 : 0; a.pad_index = pad_index;
    a.g = ConvGeom{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    a.alpha = alpha; a.beta = beta; a.zero_x = zero_x; a.zero_w = zero_w; a.wsum = wsum;
    return launch_gemm(a, cfg, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}
