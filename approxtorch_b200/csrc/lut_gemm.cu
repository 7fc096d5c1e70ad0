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
//    (i = lane + 32 j) that the lane will write out.  It arrives as ONE bulk asynchronous copy
//    (cp.async.bulk completing on an mbarrier) that overlaps the first operand gather, once per thread block.
//  * For every k-step the block STAGES the 64 table columns its 64 output channels need as 16 QUAD rows:
//    quad row p interleaves the columns of output channels p, p + 16, p + 32 and p + 48, its 8-byte entry x
//    being {T[w_p][x], T[w_p+16][x]} {T[w_p+32][x], T[w_p+48][x]}.  Building a quad row is four 16-byte
//    reads, 16 byte-permutes and eight conflict-free 8-byte writes per lane; warp p builds quad row p.
//  * The quad-row pitch is 2056 bytes (514 words, 2 mod 32).  An 8-byte shared load is served half a warp
//    at a time, and the 16 lanes of a half - one quad row each, the same activation value x (that of the
//    pixel row the half works on) - hit all 32 banks once: bank = (2 q + 2 x + {0, 1}) mod 32.  So a lookup
//    instruction costs one wavefront per 64 lookups and one instruction per 128.
//  * Each thread keeps 16 pixel rows x 4 output channels of exact integer accumulators in registers (a warp
//    32 rows x 64 channels), so staging one column (8 wavefronts) is amortised over `block_rows` (up to 512)
//    lookups.
//  * Entries are unsigned 16-bit (signed tables carry a +32768 bias removed in the epilogue).  A fetched
//    word v = lo + 65536*hi is accumulated as S0 += v and S1 += hi; the low channel's sum is
//    S0 - 65536*S1 (exact modulo 2^32 for reductions of up to 65536 steps).
//
// Scheduling is persistent stream-K.  The work is cut into units of (tile, 16-step k-chunk), tile-major with
// the column tile fastest, and dealt out in equal contiguous runs, one run per thread block (one block per SM).
// A block loads the table once and works through the tile segments of its run.  A segment that covers a
// whole tile is finished and written straight to y.  A tile that is cut between blocks is finished by
// whichever of its blocks arrives LAST: every other block parks its accumulators in its own scratch slot
// (16-byte stores in the thread's own register order, so the finisher reads them back with the same
// mapping), bumps the tile's arrival counter after a fence, and moves on; the block whose bump completes
// the count adds the parked partial sums to its own registers and runs the normal epilogue.  Nobody ever
// waits for anybody, so any grid size is safe, no reduction kernel is needed, and partial sums of whole
// tiles never touch memory.
//
// Integer-valued tables (the int16 / uint16 images) accumulate exactly in int32, so the result does not
// depend on how a tile was cut.  Tables that are not 16-bit exact take the fp32 path: lookups go to the
// transposed fp32 table in global memory (L1/L2 resident) and are summed in fp32 in ascending k inside a
// segment, and the segments of a cut tile are added in ascending k order, whoever finishes
// (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:278-281 sums ascending k, :148-163 adds its split-K
// partials in ascending order).
//
// The pixel operand is either a column matrix x[N,K,L] (L == 1: row-major A[M,K]) or the quantised
// image itself with the im2col gather done in the tile loader, so the conv never materialises the
// K/C-times larger column matrix (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:216-269
// is what it replaces).
#include "common.cuh"

namespace atb {

constexpr int kStagedCols = 64;                          // output channels per tile
constexpr int kChunk = 16;                               // k-steps per operand tile = one scheduling unit
constexpr int kQuadRows = kStagedCols / 4;               // staged quad rows per k-step
constexpr int kQuadPitch = 2056;                         // bytes per quad row (256 x 4 x uint16 + 8 B skew)
constexpr int kStageBytes = kQuadRows * kQuadPitch;      // 32896
constexpr int kMaxBlockRows = 512;
constexpr int kThreads = 512;                            // 16 warps: warp p stages quad row p
constexpr int kTableBytes = 65536 * 2;
constexpr int kMaxK = 65536;                             // longest reduction the modulo-2^32 sums keep exact
constexpr int kSmemStage = kTableBytes;
constexpr int kSmemX = kSmemStage + 2 * kStageBytes;
constexpr int kSmemW = kSmemX + 2 * kChunk * kMaxBlockRows;
constexpr int kSmemTotal = kSmemW + 2 * kChunk * kStagedCols;   // 215552 bytes
// one parked partial tile: 16 uint4 per thread (its 64 accumulators) + one int per thread (operand row sum)
constexpr int kSlotVecs = 16 * kThreads + kThreads / 4;  // in 16-byte vectors: 133120 bytes

// device-side error word of the library (0 = none); see atb_device_status
__device__ int g_device_status = 0;
constexpr int kMaxK32 = 16384;                       // reductions whose zero-point corrected sums fit 32 bits
constexpr int kStatusTableCopyTimeout = 1;
constexpr int kStatusRowsOrientationNeedsIntegerTable = 2;

struct GemmArgs {
    const uint8_t* x;
    const uint8_t* w;
    const LutImage* img;
    float* y;
    int* counters;         // arrival counter per tile, zero when the launch starts
    uint4* slots;          // two parking slots per block (first / last segment of its run), kSlotVecs each
    int units_per_cta;     // (tile, k-chunk) units per block
    long long total_units;
    int col_tiles, nchunks, block_rows;
    long long R;           // pixel rows
    int K, L, O;
    int wb_rows;           // pixel rows per weight matrix (0: one matrix for all rows)
    long long w_batch_stride;
    int tiles_per_batch;   // row tiles per weight batch (wb_rows != 0)
    int image_mode;        // 1: x is the quantised image, gather taps in the loader
    int x_xor;             // 0x80 when the image holds int8 values (idx = v + 128), else 0
    int pad_index;
    ConvGeom g;
    const float* alpha;
    const float* beta;
    const float* zero_x;
    const float* zero_w;
    const int* wsum;
    // Channels-as-rows orientation (atb_lut_conv2d_rows_fwd): the row operand is the weight matrix [channels, K], the
    // column operand the pixel matrix [pixels, K]; alpha, beta and zero_w are then indexed by ROW, wsum holds the
    // pixels' operand sums (indexed by column), and element (row, column) lands at y[n][row][l] with column = n * out_L + l.
    int rows_are_channels;
    int out_L;
};

// description of the segment a block is working on, kept in shared memory (the main loop has no register to spare)
struct SegDesc {
    int row_tile, c0, ch_beg, ch_end;
    int tile;              // tile index (arrival counter)
    int nsegs, seg;        // segments this tile is cut into (1: whole), and which of them this is
    int first_cta;         // block that holds segment 0
    int which;             // parking slot of this block used for this segment (0 / 1)
    long long next_u;
};

// Epilogue arithmetic.  Integer tables: the sum, the zero-point terms and their combination are exact integers,
// converted to fp32 once (round to nearest even), then scaled and shifted.  A signed table's sum fits 32 bits, an
// unsigned table's 33, the zero-point terms need 64.
__device__ __forceinline__ float scale_shift(float v, int o, const GemmArgs& a)
{
    // two roundings, like the separate multiply and add of the reference's dequantisation: never contracted into an
    // FMA, so that every epilogue variant of this file gives the same bits
    if (a.alpha != nullptr) v = __fmul_rn(v, __ldg(a.alpha + o));
    if (a.beta != nullptr) v = __fadd_rn(v, __ldg(a.beta + o));
    return v;
}

__device__ __forceinline__ float finalize_output(long long total, long long xsum, int o, const GemmArgs& a)
{
    float v;
    if (a.zero_x != nullptr && a.K <= kMaxK32) {
        // up to 16384 steps every term is below 2^30 in magnitude and the corrected sum below 2^31: 32-bit arithmetic
        // (wrapping on the way, exact at the end) instead of 64-bit multiplies and a 64-bit conversion
        const int zx = __float2int_rn(__ldg(a.zero_x));
        const int zw = __float2int_rn(__ldg(a.zero_w + o));
        const int ws = __ldg(a.wsum + o);
        const unsigned t32 = static_cast<unsigned>(total) - static_cast<unsigned>(zw) * static_cast<unsigned>(xsum) -
                             static_cast<unsigned>(zx) * static_cast<unsigned>(ws) +
                             static_cast<unsigned>(a.K) * static_cast<unsigned>(zx) * static_cast<unsigned>(zw);
        v = __int2float_rn(static_cast<int>(t32));
    } else if (a.zero_x != nullptr) {
        const long long zx = llrintf(__ldg(a.zero_x));
        const long long zw = llrintf(__ldg(a.zero_w + o));
        const long long ws = __ldg(a.wsum + o);
        v = __ll2float_rn(total - zw * xsum - zx * ws + static_cast<long long>(a.K) * zx * zw);
    } else if (a.K <= kMaxK32) {
        v = __int2float_rn(static_cast<int>(static_cast<unsigned>(total)));     // |sum| < 2^30: one 32-bit conversion
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
// and S1 += high half (a dot-product-accumulate that multiplies the halves by {0, 1}).
// An 8-byte shared load is served half a warp at a time, and the 16 lanes of a half (one quad row each, the
// same activation value x) hit all 32 banks once: bank = (2 q + 2 x + {0, 1}) mod 32.
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
        acc[j][1] = __dp2a_lo(v.x, 0x00000100u, acc[j][1]);
        acc[j][3] = __dp2a_lo(v.y, 0x00000100u, acc[j][3]);
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
        uint32_t v[kChunk];
        if (khw == 1) {
            // a 1x1 kernel: the reduction index is the channel, the sixteen taps lie one image plane apart
            const bool inside_px = static_cast<unsigned>(rc.ih0) < static_cast<unsigned>(a.g.H) &&
                                   static_cast<unsigned>(rc.iw0) < static_cast<unsigned>(a.g.W);
            const long long plane = static_cast<long long>(a.g.H) * a.g.W;
            const uint8_t* px = rc.base + (inside_px ? rc.ih0 * a.g.W + rc.iw0 : 0);
#pragma unroll
            for (int kk = 0; kk < kChunk; ++kk) {
                const bool inside = inside_px && (k0 + kk < kend);
                const uint32_t b = static_cast<uint32_t>(__ldg(px + (inside ? (k0 + kk) * plane : 0LL))) ^ static_cast<uint32_t>(a.x_xor);
                v[kk] = inside ? b : static_cast<uint32_t>(pad);
            }
        } else {
        int c = k0 / khw;
        const int rem = k0 - c * khw;
        int i = rem / a.g.KW;
        int j = rem - i * a.g.KW;
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
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
            xr[q] = v[4 * q] | (v[4 * q + 1] << 8) | (v[4 * q + 2] << 16) | (v[4 * q + 3] << 24);
    } else if (vec_x) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(rc.base + k0));
        const uint32_t flip = static_cast<uint32_t>(a.x_xor) * 0x01010101u;      // int8 values -> indices, 4 at a time
        xr[0] = v.x ^ flip; xr[1] = v.y ^ flip; xr[2] = v.z ^ flip; xr[3] = v.w ^ flip;
    } else {
        xr[0] = xr[1] = xr[2] = xr[3] = 0u;
#pragma unroll
        for (int kk = 0; kk < kChunk; ++kk) {
            if (k0 + kk < kend) {
                const uint32_t v = static_cast<uint32_t>(__ldg(rc.base + static_cast<long long>(k0 + kk) * a.L)) ^
                                   static_cast<uint32_t>(a.x_xor);
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

// Sum of the first `kc` of the sixteen operand bytes a thread holds for its pixel row (the zero-point correction
// needs the row sums; taking them here costs a dozen instructions per chunk instead of a shared-memory byte load per
// k-step)
__device__ __forceinline__ int chunk_sum(const uint32_t (&xr)[4], int kc)
{
    int s = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int nv = kc - 4 * q;
        uint32_t w = xr[q];
        if (nv < 4) w = nv <= 0 ? 0u : (w & ((1u << (8 * nv)) - 1u));
        s = static_cast<int>(__dp4a(w, 0x01010101u, static_cast<unsigned>(s)));
    }
    return s;
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
// The L == 1 layout is written directly (lanes span consecutive channels, the fast axis there).  For L > 1 the
// fast axis of y[n, o, l] is the pixel, so each warp turns its 32 x 64 tile around in shared memory, 32 channels
// at a time, and stores 128 contiguous bytes per channel.  The turning space is the stage / operand area, which
// every warp has left by the time the main loop's last barrier is passed; the table image stays intact for the
// block's next segment.  `active` is uniform over a warp (warps beyond the tile's rows hold nothing).
template <bool QUAD, class Total>
__device__ __forceinline__ void write_tile(const GemmArgs& a, uint8_t* smem, long long r0, long long r_end, int c0,
                                           int warp, int lane, int xsum, bool active, Total total)
{
    constexpr int NJ = QUAD ? 16 : 32;               // row slots per thread
    constexpr int NT = QUAD ? 4 : 2;                 // column slots per thread
    constexpr int TH = NT / 2;                       // column slots per 32-channel half
    const int row_base = QUAD ? (lane >> 4) * 16 : 0;        // first of this thread's rows within the warp's 32
    const int col_base = QUAD ? (lane & 15) : lane;          // first of this thread's columns within the 64
    constexpr int col_step = QUAD ? 16 : 32;
    if (!active) return;
    if constexpr (QUAD) {
        if (a.rows_are_channels) {
            long long col_off[NT];
            long long col_sum[NT];
            bool col_ok[NT];
            const bool zp = a.zero_x != nullptr;
            const long long zc = zp ? llrintf(__ldg(a.zero_x)) : 0LL;       // the column operand's (activations') zero point
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int o = c0 + col_base + col_step * t;
                col_ok[t] = o < a.O;
                const int oc = col_ok[t] ? o : 0;
                const int n = oc / a.out_L;
                col_off[t] = static_cast<long long>(n) * a.R * a.out_L + (oc - n * a.out_L);
                col_sum[t] = zp ? static_cast<long long>(__ldg(a.wsum + oc)) : 0LL;
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const long long r = r0 + warp * 32 + row_base + j;
                const long long xs = __shfl_sync(0xffffffffu, xsum, row_base + j);
                if (r >= r_end) continue;
                const long long zr = zp ? llrintf(__ldg(a.zero_w + r)) : 0LL;  // the row operand's (this channel's) zero point
                const float al = a.alpha != nullptr ? __ldg(a.alpha + r) : 1.0f;
                const float be = a.beta != nullptr ? __ldg(a.beta + r) : 0.0f;
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    if (!col_ok[t]) continue;
                    long long v = total(j, t);
                    float f;
                    if (zp && a.K <= kMaxK32) {
                        const unsigned t32 = static_cast<unsigned>(v) - static_cast<unsigned>(zc) * static_cast<unsigned>(xs) -
                                             static_cast<unsigned>(zr) * static_cast<unsigned>(col_sum[t]) +
                                             static_cast<unsigned>(a.K) * static_cast<unsigned>(zr) * static_cast<unsigned>(zc);
                        f = __int2float_rn(static_cast<int>(t32));
                    } else if (a.K <= kMaxK32) {
                        f = __int2float_rn(static_cast<int>(static_cast<unsigned>(v)));
                    } else {
                        if (zp) v = v - zc * xs - zr * col_sum[t] + static_cast<long long>(a.K) * zr * zc;
                        f = __ll2float_rn(v);
                    }
                    if (a.alpha != nullptr) f = __fmul_rn(f, al);
                    if (a.beta != nullptr) f = __fadd_rn(f, be);
                    a.y[col_off[t] + r * a.out_L] = f;
                }
            }
            return;
        }
    }
    // Integer tables with sums that fit 32 bits: what depends on the column only (zero point, its products, scale,
    // shift) is fetched once per thread and column instead of once per output element.
    const bool fast = QUAD && a.K <= kMaxK32;
    unsigned ce_zw[NT], ce_cc[NT];
    float ce_al[NT], ce_be[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        ce_zw[t] = 0u; ce_cc[t] = 0u; ce_al[t] = 1.0f; ce_be[t] = 0.0f;
        if (fast) {
            const int o = min(c0 + col_base + col_step * t, a.O - 1);
            if (a.zero_x != nullptr) {
                const unsigned zx = static_cast<unsigned>(__float2int_rn(__ldg(a.zero_x)));
                const unsigned zw = static_cast<unsigned>(__float2int_rn(__ldg(a.zero_w + o)));
                ce_zw[t] = zw;
                ce_cc[t] = static_cast<unsigned>(a.K) * zx * zw - zx * static_cast<unsigned>(__ldg(a.wsum + o));
            }
            if (a.alpha != nullptr) ce_al[t] = __ldg(a.alpha + o);
            if (a.beta != nullptr) ce_be[t] = __ldg(a.beta + o);
        }
    }
    auto fin = [&](int j, int t, int xs, int o) -> float {
        if constexpr (QUAD) {
            if (fast) {
                const unsigned v = static_cast<unsigned>(total(j, t)) - ce_zw[t] * static_cast<unsigned>(xs) + ce_cc[t];
                float f = __int2float_rn(static_cast<int>(v));
                if (a.alpha != nullptr) f = __fmul_rn(f, ce_al[t]);
                if (a.beta != nullptr) f = __fadd_rn(f, ce_be[t]);
                return f;
            }
        }
        return finalize_output(total(j, t), xs, o, a);
    };
    if (a.L == 1) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const long long r = r0 + warp * 32 + row_base + j;
            const int xs = __shfl_sync(0xffffffffu, xsum, row_base + j);
            if (r >= r_end) continue;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int o = c0 + col_base + col_step * t;
                if (o < a.O) a.y[r * a.O + o] = fin(j, t, xs, o);
            }
        }
        return;
    }
    constexpr int kPitch = 33;                         // words per channel row of the turned tile
    float* tile = reinterpret_cast<float*>(smem + kSmemStage) + warp * (32 * kPitch);
    const long long r = r0 + warp * 32 + lane;         // this lane's pixel row
    const long long n = r / a.L;
    const long long l = r - n * a.L;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int xs = __shfl_sync(0xffffffffu, xsum, row_base + j);
#pragma unroll
            for (int tt = 0; tt < TH; ++tt) {
                const int t = half * TH + tt;
                const int oc = col_base + col_step * t;            // channel within the 64
                tile[(oc - 32 * half) * kPitch + row_base + j] = (c0 + oc < a.O) ? fin(j, t, xs, c0 + oc) : 0.0f;
            }
        }
        __syncwarp();
        if (r < r_end) {
            float* dst = a.y + (n * a.O + c0 + 32 * half) * a.L + l;
            const int ncols = min(32, a.O - c0 - 32 * half);
            for (int c = 0; c < ncols; ++c) dst[static_cast<long long>(c) * a.L] = tile[c * kPitch + lane];
        }
        __syncwarp();
    }
}

// ---- cut tiles: park or finish --------------------------------------------------------------------------------
// `vec(e)` gives access to the thread's e-th group of four accumulators (e = 0..15) as a uint4.  Returns true when
// this block is the last of the tile's blocks to arrive: its registers then hold the complete sums.
// FLOAT: the partial sums are fp32 and are added in ascending segment order (deterministic whoever finishes);
// otherwise they are integers modulo 2^32 and the order does not matter.
template <bool FLOAT, class Get, class Set>
__device__ __forceinline__ bool park_or_finish(const GemmArgs& a, const volatile SegDesc* d, volatile int* s_flag,
                                               bool active, int& xsum, Get get, Set set)
{
    const int tid = threadIdx.x;
    const int nsegs = d->nsegs;
    int* ctr = a.counters + d->tile;
    if (tid == 0) {
        int seen;
        asm volatile("ld.acquire.gpu.s32 %0, [%1];" : "=r"(seen) : "l"(ctr) : "memory");
        *s_flag = (seen == nsegs - 1);                 // everybody else is already in: nothing to park
    }
    __syncthreads();
    bool last = *s_flag != 0;
    if (!last) {
        uint4* slot = a.slots + (2LL * blockIdx.x + d->which) * kSlotVecs;
        if (active) {
#pragma unroll
            for (int e = 0; e < 16; ++e) slot[e * kThreads + tid] = get(e);
            reinterpret_cast<int*>(slot + 16 * kThreads)[tid] = xsum;
        }
        __threadfence();                               // the parked sums are visible device-wide before the bump
        __syncthreads();
        if (tid == 0) *s_flag = (atomicAdd(ctr, 1) == nsegs - 1);
        __syncthreads();
        last = *s_flag != 0;
        if (!last) return false;
    }
    __threadfence();
    if (active) {
        const long long tile_u0 = static_cast<long long>(d->tile) * a.nchunks;
        const int first = d->first_cta, mine = d->seg;
        if (a.zero_x != nullptr) {
            for (int s = 0; s < nsegs; ++s) {
                if (s == mine) continue;
                const long long b = first + s;
                const uint4* slot = a.slots + (2LL * b + (tile_u0 > b * a.units_per_cta ? 1 : 0)) * kSlotVecs;
                xsum += __ldcg(reinterpret_cast<const int*>(slot + 16 * kThreads) + tid);
            }
        }
        if (!FLOAT) {
            // integer sums (modulo 2^32, any order): one segment at a time, eight of its 16-byte pieces requested
            // together so that their latencies overlap instead of adding up
            for (int s = 0; s < nsegs; ++s) {
                if (s == mine) continue;
                const long long b = first + s;
                const uint4* slot = a.slots + (2LL * b + (tile_u0 > b * a.units_per_cta ? 1 : 0)) * kSlotVecs + tid;
#pragma unroll
                for (int e0 = 0; e0 < 16; e0 += 8) {
                    uint4 p[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) p[i] = __ldcg(slot + (e0 + i) * kThreads);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        uint4 sum = get(e0 + i);
                        sum.x += p[i].x; sum.y += p[i].y; sum.z += p[i].z; sum.w += p[i].w;
                        set(e0 + i, sum);
                    }
                }
            }
        } else {
            // fp32 sums in ascending segment order whoever finishes (a rarely taken path: tables of the fp32 class
            // normally run on the kernel that keeps the table on chip)
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const uint4 own = get(e);
                uint4 sum = make_uint4(0u, 0u, 0u, 0u);
                for (int s = 0; s < nsegs; ++s) {
                    uint4 p = own;
                    if (s != mine) {
                        const long long b = first + s;
                        const uint4* slot = a.slots + (2LL * b + (tile_u0 > b * a.units_per_cta ? 1 : 0)) * kSlotVecs;
                        p = __ldcg(slot + e * kThreads + tid);
                    }
                    sum.x = __float_as_uint(__uint_as_float(sum.x) + __uint_as_float(p.x));
                    sum.y = __float_as_uint(__uint_as_float(sum.y) + __uint_as_float(p.y));
                    sum.z = __float_as_uint(__uint_as_float(sum.z) + __uint_as_float(p.z));
                    sum.w = __float_as_uint(__uint_as_float(sum.w) + __uint_as_float(p.w));
                }
                set(e, sum);
            }
        }
    }
    return true;
}

// ---- table image into shared memory: one bulk asynchronous copy completing on an mbarrier ---------------------
__device__ __forceinline__ void table_copy_start(uint8_t* smem, const LutImage* img, uint64_t* bar)
{
    const uint32_t bar_a = static_cast<uint32_t>(__cvta_generic_to_shared(bar));
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const char* src = reinterpret_cast<const char*>(img->tabTP16);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(kTableBytes) : "memory");
    constexpr int kPiece = 32768;
#pragma unroll
    for (int i = 0; i < kTableBytes / kPiece; ++i)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst + i * kPiece), "l"(src + i * kPiece), "r"(kPiece), "r"(bar_a) : "memory");
}

// Bounded wait for the copy (phase 0 of the barrier).  false: gave up.
__device__ __forceinline__ bool table_copy_wait(uint64_t* bar)
{
    const uint32_t bar_a = static_cast<uint32_t>(__cvta_generic_to_shared(bar));
    for (int i = 0; i < (1 << 20); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar_a) : "memory");
        if (ok) return true;
    }
    return false;
}

// 16-bit table classes: staged conflict-free lookups, exact integer accumulation.
// Software pipeline per k-step: issue the table reads for the NEXT step's quad row, do this step's
// lookups (which hides the latency of those reads), permute and store the next step's quad row into the
// other stage buffer, one barrier.
// Returns false when the table copy did not arrive (the block gives up).
template <bool RAGGED>
__device__ __forceinline__ bool gemm_body_int(const GemmArgs& a, uint8_t* smem, const RowCursor& rc,
                                              const uint8_t* wcol, bool vec_x, bool vec_w, int pad, int bias,
                                              long long r_end, int kbeg, int kend,
                                              const volatile SegDesc* desc, volatile int* s_flag, uint64_t* bar, bool wait_table)
{
    constexpr int TM = 32;                       // pixel rows per warp
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
    const int bm = a.block_rows;
    const bool active = !RAGGED || warp * TM < bm;

    unsigned acc[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) { acc[j][0] = 0u; acc[j][1] = 0u; acc[j][2] = 0u; acc[j][3] = 0u; }
    int xsum = 0;
    const bool want_xsum = a.zero_x != nullptr;

    uint32_t xr[4], wr[4];
    load_chunk(a, rc, wcol, vec_x, vec_w, kbeg, kend, tid, pad, xr, wr, bm);
    // thread t loads pixel row t of the tile, which is also the row whose operand sum the epilogue asks it for
    const bool sum_rows = want_xsum && tid < bm;
    if (sum_rows) xsum += chunk_sum(xr, min(kChunk, kend - kbeg));
    store_chunk(s_x, s_w, 0, tid, xr, wr, bm);
    if (wait_table) {
        const bool ok = table_copy_wait(bar);
        if (!__syncthreads_and(ok)) {
            if (tid == 0) atomicExch(&g_device_status, kStatusTableCopyTimeout);
            return false;
        }
    } else {
        __syncthreads();      // first operand tile is in shared memory
    }
    stage_quads(s_stage, s_tab, s_w, warp, lane, kThreads / 32);
    __syncthreads();

    int step = 0;
    if (RAGGED && !active) {
        // Warps beyond the tile's rows hold no accumulators: they only build their quad row of every k-step (and pass
        // the same barriers), in a loop of their own so that the working warps' loop carries no predicate.
        for (int ci = 0; ci < nch; ++ci) {
            const int k0 = kbeg + ci * kChunk;
            const int kc = min(kChunk, kend - k0);
            const int cur = ci & 1;
            const bool has_next = ci + 1 < nch;
            // the weight tile is loaded by the block's first 64 threads, which may belong to a warp without rows
            if (has_next && tid < kStagedCols) load_chunk(a, rc, wcol, vec_x, vec_w, k0 + kChunk, kend, tid, pad, xr, wr, bm);
            for (int kk = 0; kk < kc; ++kk, ++step) {
                if (has_next && kk == 4 && tid < kStagedCols) store_chunk(s_x, s_w, cur ^ 1, tid, xr, wr, bm);
                const uint8_t* wstep = s_w + (cur * kChunk + kk) * kStagedCols;
                const uint8_t* wnext = nullptr;
                if (kk + 1 < kc) wnext = wstep + kStagedCols;
                else if (has_next) wnext = s_w + ((cur ^ 1) * kChunk) * kStagedCols;
                if (wnext != nullptr) {
                    QuadWords v;
                    fetch_quad(s_tab, wnext, warp, lane, v);
                    store_quad(s_stage + ((step + 1) & 1) * kStageBytes, warp, lane, v);
                }
                __syncthreads();
            }
        }
    } else {
        for (int ci = 0; ci < nch; ++ci) {
            const int k0 = kbeg + ci * kChunk;
            const int kc = min(kChunk, kend - k0);
            const int cur = ci & 1;
            const bool has_next = ci + 1 < nch;
            if (has_next) {
                load_chunk(a, rc, wcol, vec_x, vec_w, k0 + kChunk, kend, tid, pad, xr, wr, bm);
                if (sum_rows) xsum += chunk_sum(xr, min(kChunk, kend - k0 - kChunk));
            }
            for (int kk = 0; kk < kc; ++kk, ++step) {
                if (has_next && kk == 4) store_chunk(s_x, s_w, cur ^ 1, tid, xr, wr, bm);
                const uint8_t* xrow = s_x + (cur * kChunk + kk) * kMaxBlockRows + warp * TM;
                const uint8_t* wstep = s_w + (cur * kChunk + kk) * kStagedCols;
                const uint8_t* wnext = nullptr;
                if (kk + 1 < kc) wnext = wstep + kStagedCols;
                else if (has_next) wnext = s_w + ((cur ^ 1) * kChunk) * kStagedCols;
                uint8_t* stage_next = s_stage + ((step + 1) & 1) * kStageBytes;
                const uint8_t* stage_cur = s_stage + (step & 1) * kStageBytes;

                QuadWords v;
                if (wnext != nullptr) fetch_quad(s_tab, wnext, warp, lane, v);
                lookup_step(stage_cur, xrow + h * 16, q, acc);
                if (wnext != nullptr) store_quad(stage_next, warp, lane, v);
                __syncthreads();
            }
        }
    }
    long long ksteps = kend - kbeg;
    if (desc->nsegs > 1) {
        const bool finish = park_or_finish<false>(
            a, desc, s_flag, active, xsum,
            [&](int e) { return make_uint4(acc[e][0], acc[e][1], acc[e][2], acc[e][3]); },
            [&](int e, const uint4& s) { acc[e][0] = s.x; acc[e][1] = s.y; acc[e][2] = s.z; acc[e][3] = s.w; });
        if (!finish) return true;
        ksteps = a.K;
    }
    const long long remove = static_cast<long long>(bias) * ksteps;     // +32768 per looked-up entry of a signed table
    // per word: acc[j][2u] holds sum(lo) + 65536 * sum(hi) modulo 2^32, acc[j][2u + 1] holds sum(hi)
    auto total = [&](int j, int t) -> long long {
        const int u = (t >> 1) * 2;
        const unsigned v = (t & 1) == 0 ? acc[j][u] - (acc[j][u + 1] << 16) : acc[j][u + 1];
        return static_cast<long long>(v) - remove;
    };
    // the tile coordinates were not kept in registers across the main loop; read them back
    const int tpb = a.tiles_per_batch;
    const int row_tile = desc->row_tile;
    const long long r0 = a.wb_rows > 0 ? static_cast<long long>(row_tile / tpb) * a.wb_rows + static_cast<long long>(row_tile % tpb) * bm
                                       : static_cast<long long>(row_tile) * bm;
    write_tile<true>(a, smem, r0, r_end, desc->c0, warp, lane, xsum, active, total);
    return true;
}

// Tables that are not 16-bit exact: lookups from the transposed fp32 table in global memory,
// fp32 accumulation in ascending k.
template <bool RAGGED>
__device__ __forceinline__ bool gemm_body_f32(const GemmArgs& a, uint8_t* smem, const RowCursor& rc,
                                              const uint8_t* wcol, bool vec_x, bool vec_w, int pad,
                                              long long r_end, int kbeg, int kend,
                                              const volatile SegDesc* desc, volatile int* s_flag)
{
    constexpr int TM = 32;
    uint8_t* s_x = smem + kSmemX;
    uint8_t* s_w = smem + kSmemW;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int nch = (kend - kbeg + kChunk - 1) / kChunk;
    const int bm = a.block_rows;
    const bool active = !RAGGED || warp * TM < bm;

    float acc[TM][2];
#pragma unroll
    for (int j = 0; j < TM; ++j) { acc[j][0] = 0.0f; acc[j][1] = 0.0f; }
    int xsum = 0;
    const bool want_xsum = a.zero_x != nullptr;

    uint32_t xr[4], wr[4];
    load_chunk(a, rc, wcol, vec_x, vec_w, kbeg, kend, tid, pad, xr, wr, bm);
    store_chunk(s_x, s_w, 0, tid, xr, wr, bm);
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
            if (want_xsum) xsum += static_cast<int>(xrow[lane]);
            if (active) lookup_step_f32<TM>(a.img->tabT32, wstep, xrow, lane, acc);
        }
        __syncthreads();
    }
    if (desc->nsegs > 1) {
        const bool finish = park_or_finish<true>(
            a, desc, s_flag, active, xsum,
            [&](int e) {
                return make_uint4(__float_as_uint(acc[2 * e][0]), __float_as_uint(acc[2 * e][1]),
                                  __float_as_uint(acc[2 * e + 1][0]), __float_as_uint(acc[2 * e + 1][1]));
            },
            [&](int e, const uint4& s) {
                acc[2 * e][0] = __uint_as_float(s.x); acc[2 * e][1] = __uint_as_float(s.y);
                acc[2 * e + 1][0] = __uint_as_float(s.z); acc[2 * e + 1][1] = __uint_as_float(s.w);
            });
        if (!finish) return true;
    }
    const int tpb = a.tiles_per_batch;
    const int row_tile = desc->row_tile;
    const long long r0 = a.wb_rows > 0 ? static_cast<long long>(row_tile / tpb) * a.wb_rows + static_cast<long long>(row_tile % tpb) * bm
                                       : static_cast<long long>(row_tile) * bm;
    write_tile<false>(a, smem, r0, r_end, desc->c0, warp, lane, xsum, active,
                      [&](int j, int t) { return acc[j][t]; });
    return true;
}

// One tile segment: rows of row tile `row_tile`, the 64 output channels from c0, k-chunks [ch_beg, ch_end).
template <bool RAGGED>
__device__ __forceinline__ bool run_segment(const GemmArgs& a, uint8_t* smem, int cls, const volatile SegDesc* desc,
                                            volatile int* s_flag, uint64_t* bar, bool wait_table)
{
    const int tid = threadIdx.x;
    const int bm = a.block_rows;
    const int row_tile = desc->row_tile;
    const int c0 = desc->c0;

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
    const int kbeg = desc->ch_beg * kChunk;
    const int kend = min(a.K, desc->ch_end * kChunk);

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
    if (cls == LUT_F32 && a.rows_are_channels) {
        // the channels-as-rows epilogue exists for the integer classes only: refuse loudly instead of writing a
        // differently laid out result
        if (tid == 0) atomicExch(&g_device_status, kStatusRowsOrientationNeedsIntegerTable);
        return false;
    }
    if (cls != LUT_F32)
        return gemm_body_int<RAGGED>(a, smem, rc, wcol, vec_x, vec_w, pad, cls == LUT_I16 ? 32768 : 0, r_end, kbeg, kend,
                                     desc, s_flag, bar, wait_table);
    return gemm_body_f32<RAGGED>(a, smem, rc, wcol, vec_x, vec_w, pad, r_end, kbeg, kend, desc, s_flag);
}

// 16 warps per block, 32 pixel rows per warp (one thread per row loads the operand tiles, 64 accumulators per
// thread).  RAGGED: tiles are shorter than 512 rows and the warps beyond them only help with the staging.
template <bool RAGGED>
__global__ void __launch_bounds__(kThreads, 1) lut_gemm_kernel(const GemmArgs a)
{
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ SegDesc s_desc;
    __shared__ int s_flag;
    const int tid = threadIdx.x;
    const int cls = lut_class_of(a.img);
    long long u = static_cast<long long>(blockIdx.x) * a.units_per_cta;
    const long long u_end = min(a.total_units, u + a.units_per_cta);
    if (u >= u_end) return;
    // The image holds the table as the lookups want it (signed entries biased by +32768, so every lookup is an
    // unsigned 16-bit load); it is copied into shared memory untouched while the first operand tile is gathered.
    if (cls != LUT_F32 && tid == 0) table_copy_start(smem, a.img, &s_bar);
    bool wait_table = cls != LUT_F32;
    while (true) {
        if (tid == 0) {
            const int n = a.nchunks;
            const int U = a.units_per_cta;
            const int tile = static_cast<int>(u / n);
            const int ch_beg = static_cast<int>(u - static_cast<long long>(tile) * n);
            const int ch_end = static_cast<int>(min(static_cast<long long>(n), ch_beg + (u_end - u)));
            const int row_tile = tile / a.col_tiles;
            const long long t0 = static_cast<long long>(tile) * n;
            const int first = static_cast<int>(t0 / U);
            const int last = static_cast<int>((t0 + n - 1) / U);
            s_desc.row_tile = row_tile;
            s_desc.c0 = (tile - row_tile * a.col_tiles) * kStagedCols;
            s_desc.ch_beg = ch_beg;
            s_desc.ch_end = ch_end;
            s_desc.tile = tile;
            s_desc.nsegs = last - first + 1;
            s_desc.seg = static_cast<int>(blockIdx.x) - first;
            s_desc.first_cta = first;
            s_desc.which = t0 > static_cast<long long>(blockIdx.x) * U ? 1 : 0;
            s_desc.next_u = u + (ch_end - ch_beg);
        }
        __syncthreads();
        if (!run_segment<RAGGED>(a, smem, cls, &s_desc, &s_flag, &s_bar, wait_table)) return;
        wait_table = false;
        u = const_cast<const volatile SegDesc*>(&s_desc)->next_u;
        __syncthreads();             // everybody is done with the description and the turning space
        if (u >= u_end) break;
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

// ---- host side: the plan -----------------------------------------------------------------------------------------
// Modelled duration of a block that works through `units` k-chunks cut into `segs` tile segments, in k-steps:
// every segment pays a prologue (first operand gather, first staging) and an epilogue (finish and store, or
// park), a block whose run ends inside a tile also pays for parking / collecting the partial sums.
static double run_cost(long long units, long long segs, bool cut)
{
    constexpr double kPerSegment = 10.0, kExchange = 6.0, kPerBlock = 6.0;
    return static_cast<double>(units) * kChunk + kPerSegment * static_cast<double>(segs) + (cut ? kExchange : 0.0) + kPerBlock;
}

struct FullPlan {
    int block_rows, tiles_per_batch, col_tiles, nchunks, ctas, units_per_cta, cut;
    long long row_tiles, tiles, total_units;
    size_t counter_bytes, scratch_bytes;
};

static int make_plan(long long R, int K, int O, int wb_rows, int cfg, FullPlan* p)
{
    ATB_REQUIRE(p != nullptr, "plan is null");
    ATB_REQUIRE(R >= 0 && K >= 0 && O >= 0 && wb_rows >= 0, "negative dimension");
    ATB_REQUIRE(K <= kMaxK, "reductions longer than 65536 steps are not supported");
    ATB_REQUIRE(wb_rows == 0 || R % wb_rows == 0, "rows must be a multiple of wb_rows");
    const int sms = sm_count();
    const long long span = wb_rows > 0 ? wb_rows : R;
    int bm = 0, forced = 0;
    if (cfg >= 0) { bm = cfg & 0xffff; forced = (cfg >> 16) & 0xff; }
    if (bm != 0) {
        ATB_REQUIRE(bm % 32 == 0 && bm >= 32 && bm <= kMaxBlockRows, "cfg: block rows must be a multiple of 32 up to 512");
    } else {
        // Full 512-row tiles whenever there are that many rows.  A k-step costs a block about 0.43 us + 0.023 us per 32
        // rows (measured: the staging of the 64 columns and the barrier dominate), so a shorter tile is barely
        // cheaper than a full one and equalising tile heights gains nothing; only operands with fewer than 512 rows
        // get a shorter tile (whose idle warps then only help with the staging).
        bm = static_cast<int>(span >= kMaxBlockRows ? kMaxBlockRows : (span > 0 ? (span + 31) / 32 * 32 : 32));
    }
    const int tpb = wb_rows > 0 ? ceil_div(wb_rows, bm) : 0;
    const long long rt = wb_rows > 0 ? (R / wb_rows) * tpb : (R + bm - 1) / bm;
    const int ct = ceil_div(O > 0 ? O : 1, kStagedCols);
    const long long tiles = rt * ct;
    const int nchunks = K > 0 ? ceil_div(K, kChunk) : 1;
    const long long total = tiles * nchunks;
    ATB_REQUIRE(tiles <= 2147483647LL / 2, "too many tiles");
    long long units = nchunks;
    if (total > 0) {
        if (forced == 1) {                                   // whole tiles only
            units = static_cast<long long>(nchunks) * ((tiles + sms - 1) / sms);
        } else if (forced > 1) {                             // every tile cut into `forced` segments
            units = ceil_div(nchunks, forced);
        } else {
            // Equal runs for p = 1 .. #SM blocks; the cheapest modelled run wins, fewer blocks on a tie.  Runs of
            // whole tiles are among the candidates (p such that the run length is a multiple of the tile's chunks).
            double best = 1e300;
            for (long long pblocks = 1; pblocks <= sms && pblocks <= total; ++pblocks) {
                for (int whole = 0; whole < 2; ++whole) {
                    long long u = (total + pblocks - 1) / pblocks;
                    if (whole) u = (u + nchunks - 1) / nchunks * nchunks;
                    const bool cut = u % nchunks != 0;
                    const long long segs = cut ? (u - 1) / nchunks + 2 : u / nchunks;
                    const double c = run_cost(u, segs, cut);
                    if (c < best - 1e-9) { best = c; units = u; }
                }
            }
        }
    }
    if (units < 1) units = 1;
    ATB_REQUIRE(units <= 2147483647LL, "run too long");
    const long long ctas = total > 0 ? (total + units - 1) / units : 0;
    ATB_REQUIRE(ctas <= 2147483647LL, "too many blocks");
    p->block_rows = bm;
    p->tiles_per_batch = tpb;
    p->col_tiles = ct;
    p->nchunks = nchunks;
    p->row_tiles = rt;
    p->tiles = tiles;
    p->total_units = total;
    p->units_per_cta = static_cast<int>(units);
    p->ctas = static_cast<int>(ctas);
    p->cut = (total > 0 && units % nchunks != 0) ? 1 : 0;
    p->counter_bytes = p->cut ? (static_cast<size_t>(tiles) * 4u + 255u) / 256u * 256u : 0u;
    p->scratch_bytes = p->cut ? p->counter_bytes + 2u * static_cast<size_t>(ctas) * kSlotVecs * 16u : 0u;
    return ATB_OK;
}

template <bool RAGGED>
static int launch_one(int ctas, const GemmArgs& a, cudaStream_t stream)
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
        e = cudaFuncSetAttribute(lut_gemm_kernel<RAGGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        attr_set[dev] = true;
    }
    lut_gemm_kernel<RAGGED><<<ctas, kThreads, kSmemTotal, stream>>>(a);
    return check_launch("lut_gemm_kernel");
}

static int launch_gemm(GemmArgs a, int cfg, void* scratch, size_t scratch_bytes, cudaStream_t stream)
{
    if (a.R == 0 || a.O == 0) return ATB_OK;
    if (a.K == 0) {
        lut_gemm_empty_k_kernel<<<grid_for(a.R * a.O, 256, 4096), 256, 0, stream>>>(a);
        return check_launch("lut_gemm_empty_k_kernel");
    }
    if (cfg >= 0 && ((cfg >> 24) & 1) && a.wb_rows == 0) {
        // The caller knows the table is of the fp32 class (atb_lut_image_class): whole-reduction tiles on the kernel
        // that keeps the fp32 table on chip, half in each block of a two-block cluster.
        PairFwdParams p{};
        p.x = a.x; p.w = a.w; p.tab = a.img->tabTP32; p.y = a.y;
        p.R = a.R; p.K = a.K; p.L = a.L; p.O = a.O;
        p.image_mode = a.image_mode; p.x_xor = a.x_xor; p.pad_index = a.pad_index; p.g = a.g;
        p.alpha = a.alpha; p.beta = a.beta; p.zero_x = a.zero_x; p.zero_w = a.zero_w; p.wsum = a.wsum;
        return pair_forward_launch(p, (cfg >> 25) & 1, stream);
    }
    FullPlan plan;
    int rc = make_plan(a.R, a.K, a.O, a.wb_rows, cfg, &plan);
    if (rc != ATB_OK) return rc;
    if (plan.scratch_bytes > 0) {
        if (scratch == nullptr || scratch_bytes < plan.scratch_bytes) {
            set_error("this plan cuts tiles between blocks and needs %zu bytes of scratch, got %zu", plan.scratch_bytes, scratch_bytes);
            return ATB_ERR_SCRATCH;
        }
        ATB_REQUIRE(aligned_to(scratch, 16), "scratch must be 16-byte aligned");
        // arrival counters start at zero; the parking slots need no initialisation (written before they are read)
        cudaError_t e = cudaMemsetAsync(scratch, 0, plan.counter_bytes, stream);
        if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        a.counters = static_cast<int*>(scratch);
        a.slots = reinterpret_cast<uint4*>(static_cast<char*>(scratch) + plan.counter_bytes);
    }
    a.block_rows = plan.block_rows;
    a.tiles_per_batch = plan.tiles_per_batch;
    a.col_tiles = plan.col_tiles;
    a.nchunks = plan.nchunks;
    a.units_per_cta = plan.units_per_cta;
    a.total_units = plan.total_units;
    return plan.block_rows == kMaxBlockRows ? launch_one<false>(plan.ctas, a, stream) : launch_one<true>(plan.ctas, a, stream);
}

}  // namespace atb

using namespace atb;

extern "C" int atb_lut_gemm_plan(long long R, int K, int O, int wb_rows, int cfg, atb_gemm_plan* plan)
{
    ATB_REQUIRE(plan != nullptr, "plan is null");
    FullPlan p;
    const int rc = make_plan(R, K, O, wb_rows, cfg, &p);
    if (rc != ATB_OK) return rc;
    if (cfg >= 0 && ((cfg >> 24) & 1) && wb_rows == 0) { p.cut = 0; p.scratch_bytes = 0; }     // fp32-class kernel: whole reductions
    plan->block_rows = p.block_rows;
    plan->blocks = p.ctas;
    plan->units_per_block = p.units_per_cta;
    plan->chunks_per_tile = p.nchunks;
    plan->cut_tiles = p.cut;
    plan->scratch_bytes = p.scratch_bytes;
    return ATB_OK;
}

extern "C" int atb_lut_image_class(const void* lut_image, int* cls /*host*/, void* stream)
{
    ATB_REQUIRE(lut_image != nullptr && cls != nullptr, "null pointer");
    int flags[4] = {0, 0, 0, 0};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(flags, lut_image, sizeof(flags), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { set_error("atb_lut_image_class: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    *cls = flags[0] == 0 ? LUT_I16 : (flags[1] == 0 ? LUT_U16 : LUT_F32);
    return ATB_OK;
}

extern "C" int atb_device_status(int* status /*host*/)
{
    ATB_REQUIRE(status != nullptr, "status is null");
    cudaError_t e = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
    if (e != cudaSuccess) { set_error("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    return ATB_OK;
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
// Partial sums of tiles that are cut between blocks normally go to a caller-supplied scratch buffer.  Some hosts
// of this library cannot provide one: code running inside a CUDA-graph capture or under a memory pool that
// forbids new allocations, and bindings from runtimes whose tensors cannot be created from inside an operator
// call.  For them the library carries its own fixed scratch area in device global memory.  It exists once per
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
    FullPlan plan;
    int rc = make_plan(static_cast<long long>(N) * L, K, O, wb_rows, cfg, &plan);
    if (rc != ATB_OK) return rc;
    if (plan.scratch_bytes > ATB_STATIC_SCRATCH_BYTES) {
        set_error("this shape's plan needs %zu bytes of scratch but the built-in area holds %zu; "
                  "use atb_lut_bgemm_fwd with a caller buffer, or choose a plan without cut tiles through cfg",
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
    ATB_REQUIRE(K <= kMaxK, "C*kh*kw above 65536 is not supported");
    ATB_REQUIRE(y != nullptr && (K == 0 || (x != nullptr && w != nullptr)), "null operand");
    int rc = check_epilogue(zero_x, zero_w, wsum);
    if (rc != ATB_OK) return rc;
    GemmArgs a{};
    a.x = static_cast<const uint8_t*>(x); a.w = w; a.img = static_cast<const LutImage*>(lut_image); a.y = y;
    a.L = OH * OW; a.R = static_cast<long long>(N) * a.L; a.K = static_cast<int>(K); a.O = O;
    a.wb_rows = 0; a.w_batch_stride = 0;
    a.image_mode = 1; a.x_xor = (dtype == ATB_I8) ? 0x80 : 0; a.pad_index = pad_index;
    a.g = ConvGeom{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    if (H == 1 && W == 1 && kh == 1 && kw == 1 && ph == 0 && pw == 0) {
        // A 1x1 image under a 1x1 kernel is a plain matrix product (a fully connected layer): [N, C] rows that are
        // contiguous along the reduction, read 16 bytes at a time by the column-mode loader instead of tap by tap.
        a.image_mode = 0; a.L = 1; a.R = N;
    }
    a.alpha = alpha; a.beta = beta; a.zero_x = zero_x; a.zero_w = zero_w; a.wsum = wsum;
    return launch_gemm(a, cfg, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

// ---- channels as rows ------------------------------------------------------------------------------------------
// pix[(n * L + l) * K + k]: the operand index of tap k of output pixel (n, l), or the pad value; pixsum[p] = sum_k pix[p, k]
template <int DT>
__global__ void pixel_rows_kernel(const void* __restrict__ x, uint8_t* __restrict__ pix, int* __restrict__ pixsum,
                                  ConvGeom g, int pad_index, const float* __restrict__ zero_x)
{
    const int L = g.OH * g.OW, K = g.C * g.KH * g.KW, khw = g.KH * g.KW;
    const long long p = blockIdx.x;
    const int n = static_cast<int>(p / L);
    const int l = static_cast<int>(p - static_cast<long long>(n) * L);
    const int oh = l / g.OW, ow = l - oh * g.OW;
    const int pad = pad_index >= 0 ? pad_index : min(255, max(0, static_cast<int>(llrintf(__ldg(zero_x)))));
    const long long base = static_cast<long long>(n) * g.C * g.H * g.W;
    int sum = 0;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const int c = k / khw, rem = k - c * khw;
        const int i = rem / g.KW, j = rem - i * g.KW;
        const int ih = oh * g.SH - g.PH + i * g.DH, iw = ow * g.SW - g.PW + j * g.DW;
        int idx = pad;
        if (static_cast<unsigned>(ih) < static_cast<unsigned>(g.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(g.W))
            idx = index_of<DT>(x, base + (static_cast<long long>(c) * g.H + ih) * g.W + iw);
        pix[p * K + k] = static_cast<uint8_t>(idx);
        sum += idx;
    }
    if (pixsum != nullptr) {
        __shared__ int part[32];
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x < 32) {
            int v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0;
            for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
            if (threadIdx.x == 0) pixsum[p] = v;
        }
    }
}

// The same for a 1x1 kernel without padding: a transposition [C][pixels] -> [pixels][C].  One block turns 32 pixels x
// 256 channels around through shared memory (32 bytes read along the pixels, 32 bytes written along the channels) and
// adds its share of the pixels' sums to pixsum, which the caller has zeroed.
template <int DT>
__global__ void __launch_bounds__(256) pixel_rows_1x1_kernel(const void* __restrict__ x, uint8_t* __restrict__ pix,
                                                             int* __restrict__ pixsum, ConvGeom g, long long P)
{
    __shared__ uint8_t tile[32][33];
    const int L = g.OH * g.OW, C = g.C;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
    const long long p0 = static_cast<long long>(blockIdx.x) * 32;
    // the pixel this thread reads for
    const long long pr = p0 + tx;
    const bool pr_ok = pr < P;
    long long src = 0;
    if (pr_ok) {
        const int n = static_cast<int>(pr / L);
        const int l = static_cast<int>(pr - static_cast<long long>(n) * L);
        const int oh = l / g.OW, ow = l - oh * g.OW;
        src = (static_cast<long long>(n) * C * g.H + oh * g.SH) * g.W + ow * g.SW;
    }
    const long long plane = static_cast<long long>(g.H) * g.W;
    int sums[4] = {0, 0, 0, 0};                                          // pixels ty + 8 i, this thread's channels
    const int c_end = min(C, (static_cast<int>(blockIdx.y) + 1) * 256);
    for (int c0 = blockIdx.y * 256; c0 < c_end; c0 += 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + ty + 8 * i;
            tile[ty + 8 * i][tx] = (pr_ok && c < C) ? static_cast<uint8_t>(index_of<DT>(x, src + c * plane)) : static_cast<uint8_t>(0);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long pw_ = p0 + ty + 8 * i;
            const int c = c0 + tx;
            if (pw_ < P && c < C) {
                const uint8_t v = tile[tx][ty + 8 * i];
                pix[pw_ * C + c] = v;
                sums[i] += v;
            }
        }
        __syncthreads();
    }
    if (pixsum != nullptr) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int v = sums[i];
            for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
            const long long pw_ = p0 + ty + 8 * i;
            if (tx == 0 && pw_ < P) atomicAdd(pixsum + pw_, v);
        }
    }
}

extern "C" int atb_pixel_rows_u8(const void* x, int dtype, int N, int C, int H, int W, int kh, int kw, int sh, int sw,
                                 int ph, int pw, int dh, int dw, int pad_index, const float* zero_x,
                                 uint8_t* pix, int* pixsum, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0, "negative dimension");
    ATB_REQUIRE(dtype == ATB_I8 || dtype == ATB_U8, "image must be int8 values or uint8 indices");
    ATB_REQUIRE(pad_index >= -1 && pad_index <= 255, "pad_index out of range");
    ATB_REQUIRE(pad_index >= 0 || zero_x != nullptr, "pad_index -1 takes the pad value from zero_x, which is null");
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw, &OH, &OW), "conv geometry yields empty output");
    const long long P = static_cast<long long>(N) * OH * OW;
    const long long K = static_cast<long long>(C) * kh * kw;
    if (P == 0 || K == 0) return ATB_OK;
    ATB_REQUIRE(x != nullptr && pix != nullptr, "null pointer");
    ATB_REQUIRE(P <= 2147483647LL && K <= kMaxK, "dimensions too large");
    const ConvGeom g{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, OH, OW};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (kh == 1 && kw == 1 && ph == 0 && pw == 0) {
        if (pixsum != nullptr) {
            cudaError_t e = cudaMemsetAsync(pixsum, 0, static_cast<size_t>(P) * sizeof(int), s);
            if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        }
        const dim3 grid(static_cast<unsigned>((P + 31) / 32), static_cast<unsigned>((C + 255) / 256));
        if (dtype == ATB_I8) pixel_rows_1x1_kernel<ATB_I8><<<grid, 256, 0, s>>>(x, pix, pixsum, g, P);
        else pixel_rows_1x1_kernel<ATB_U8><<<grid, 256, 0, s>>>(x, pix, pixsum, g, P);
        return check_launch("pixel_rows_1x1_kernel");
    }
    const int threads = K >= 256 ? 256 : 128;
    if (dtype == ATB_I8) pixel_rows_kernel<ATB_I8><<<static_cast<unsigned>(P), threads, 0, s>>>(x, pix, pixsum, g, pad_index, zero_x);
    else pixel_rows_kernel<ATB_U8><<<static_cast<unsigned>(P), threads, 0, s>>>(x, pix, pixsum, g, pad_index, zero_x);
    return check_launch("pixel_rows_kernel");
}

extern "C" int atb_lut_gemm_rows_plan(int O, int K, long long P, int cfg, atb_gemm_plan* plan)
{
    ATB_REQUIRE(P >= 0 && P <= 2147483647LL, "pixel count out of range");
    return atb_lut_gemm_plan(O, K, static_cast<int>(P), 0, cfg, plan);
}

extern "C" int atb_lut_conv2d_rows_fwd(const uint8_t* w, const uint8_t* pix, const void* lut_image_t, float* y,
                                       int O, int K, long long P, int L,
                                       const float* alpha, const float* beta, const float* zero_x,
                                       const float* zero_w, const int* pixsum,
                                       int cfg, void* scratch, size_t scratch_bytes, void* stream)
{
    ATB_REQUIRE(O >= 0 && K >= 1 && P >= 0 && L >= 1, "negative dimension or empty reduction");
    ATB_REQUIRE(P <= 2147483647LL && P % L == 0, "pixel count must be a multiple of L below 2^31");
    ATB_REQUIRE(K <= kMaxK, "reductions longer than 65536 steps are not supported");
    ATB_REQUIRE(lut_image_t != nullptr, "lut_image is null");
    ATB_REQUIRE(cfg < 0 || ((cfg >> 24) & 1) == 0, "tables of the fp32 class are not served in this orientation");
    if (O == 0 || P == 0) return ATB_OK;
    ATB_REQUIRE(y != nullptr && (K == 0 || (w != nullptr && pix != nullptr)), "null operand");
    int rc = check_epilogue(zero_x, zero_w, pixsum);
    if (rc != ATB_OK) return rc;
    GemmArgs a{};
    a.x = w; a.w = pix; a.img = static_cast<const LutImage*>(lut_image_t); a.y = y;
    a.R = O; a.K = K; a.L = 1; a.O = static_cast<int>(P);
    a.wb_rows = 0; a.w_batch_stride = 0;
    a.image_mode = 0; a.x_xor = 0; a.pad_index = 0;
    a.alpha = alpha; a.beta = beta; a.zero_x = zero_x; a.zero_w = zero_w; a.wsum = pixsum;
    a.rows_are_channels = 1; a.out_L = L;
    return launch_gemm(a, cfg, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}
