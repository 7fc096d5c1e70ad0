// Custom-pair gradient backward: one surrogate derivative per (x, w) pair, two 256 x 256 fp32 tables.
//
//   grad_x[n,k,l] = sum_o dY[n,o,l] * DX[x[n,k,l]][w[o,k]]
//   grad_w[o,k]   = sum_{n,l} dY[n,o,l] * DW[x[n,k,l]][w[o,k]]
//
// Both are the forward LUT GEMM's access pattern - every (pixel row r, channel o, reduction step k) triple looks
// one table entry up - with a multiply by dY[r, o] and a different sum, so both run on the forward kernel's
// machinery (approxtorch/backend/csrc/cuda/bgemm_custom_grad_optimize.cu:30-205 gathers from the 256 KB table in
// global memory instead, one uncoalesced 4-byte read per lookup):
//
//  * The fp32 table (256 KB) does not fit one SM's shared memory next to the staging buffers, so it is held by a
//    CLUSTER OF TWO thread blocks, 128 table rows (128 KB) each, copied in once per block by one bulk asynchronous
//    copy; a block reads the other half through distributed shared memory (ld.shared::cluster).  (With the
//    cluster switched off the staging reads come from global memory / L2 instead.)
//  * Per k-step a block stages the 32 table columns T[w[o,k]][.] of its 32 output channels as 8 QUAD rows: quad
//    row q interleaves channels q, q+8, q+16, q+24, so its 16-byte entry x is one lookup for four channels.  The
//    quad-row pitch is 4112 bytes (1028 words, 4 mod 32): a 16-byte shared load is served a quarter warp at a
//    time, and the 8 lanes of a quarter - one quad row each, the same pixel row, hence the same x - cover all 32
//    banks once.  Lookups are conflict-free whatever the operands are.
//  * Lane (g, q) of a warp owns 8 pixel rows x 4 channels; its 32 dY values stay in registers for the whole run
//    of k-steps.  grad_w: the products are summed over the thread's rows, then over the warp's four row groups
//    by a three-shuffle transposing reduction (lane c ends up with channel c), then over the 16 warps through a
//    double-buffered shared array that one warp drains during the next k-step; the 32 sums of a k-step are added
//    to grad_w[o, k] (fp32 atomics: other blocks hold other pixel rows of the same sum).
//    grad_x: the products are summed over the thread's 4 channels, then over the quarter warp's 8 quad rows by a
//    seven-shuffle transposing reduction (lane r ends up with pixel row r), giving grad_x[r, k] for 32 channels;
//    the block passes over the channel tiles in turn and accumulates in place (it owns its rows and k range, so
//    the result is deterministic).  With the image form the value goes to the image pixel the tap came from
//    (fp32 atomics, the fold of approxtorch/nn/bgemm_int8.py:116-118 done in the kernel), so no [N,K,L] column
//    gradient is ever written.
//  * Work is cut into (tile, 16-step k-chunk) units dealt out in equal contiguous runs, one per block; k-steps are
//    independent outputs here, so cutting along k costs nothing.
#include "common.cuh"

namespace atb {

constexpr int PS = 32;                      // staged channels per tile
constexpr int PQ = 512;                     // pixel rows per tile
constexpr int PThreads = 512;
constexpr int PChunk = 16;                  // k-steps per operand tile
constexpr int PQuadRows = PS / 4;           // 8
constexpr int PPitch = 4112;                // bytes per quad row: 256 x 16 B + 16 B skew
constexpr int PStageBytes = PQuadRows * PPitch;      // 32896
constexpr int PTabHalf = 128 * 256 * 4;     // 131072: half of the table
constexpr int PSmemStage = PTabHalf;
constexpr int PSmemX = PSmemStage + 2 * PStageBytes;
constexpr int PSmemW = PSmemX + 2 * PChunk * PQ;
constexpr int PSmemRed = PSmemW + 2 * PChunk * PS;
constexpr int PSmemTotal = PSmemRed + 2 * 16 * PS * 4;     // 218368 bytes

__device__ int g_pair_status = 0;           // 1: a block gave up waiting for its half of the table

struct PairArgs {
    const uint8_t* x;         // [N,K,L] LUT indices, or the quantised image [N,C,H,W] (image_mode)
    const uint8_t* w;         // [O,K] LUT indices
    const float* dy;          // [N,O,L]
    const float* tab;         // prepared table: [w][x permuted], see pair_table_prepare_kernel
    float* out;               // grad_w [O,K] | grad_x [N,K,L] | grad wrt the image [N,C,H,W]
    long long R;              // pixel rows N*L
    int K, L, O;
    int image_mode, x_xor, pad_index;
    ConvGeom g;
    int row_tiles, ch_tiles, nchunks;
    int units_per_cta;
    long long total_units;
};

// ---- table image: out[w][h*128 + 4*l + e] = tab[x = h*128 + l + 32*e][w]  (tab row-major [x][w]) ------------------
// Transposed (the staging reads columns of the table) and x-permuted so that lane l of a staging warp gets the
// four entries x = l, l+32, l+64, l+96 of its half-row with one 16-byte load and then writes consecutive lanes to
// consecutive 16-byte slots.
__global__ void pair_table_prepare_kernel(const float* __restrict__ tab, float* __restrict__ out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;       // i = x * 256 + w: coalesced reads
    const int x = i >> 8, w = i & 255;
    const int h = x >> 7, xl = x & 127;
    out[(w << 8) + (h << 7) + ((xl & 31) << 2) + (xl >> 5)] = tab[i];
}

// ---- cluster helpers ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ int ld_cluster_s32(uint32_t addr)
{
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// This block's half of the table (cluster rank r holds rows 128 r .. 128 r + 127): one bulk asynchronous copy with a
// bounded wait; both blocks of the cluster then meet, so that each knows the other's half is in place and learns
// whether it arrived.  Returns false (and raises the status word) when either half is missing.
template <bool CLUSTER>
__device__ __forceinline__ bool table_half_load(const float* tab, uint32_t s_tab_addr, uint64_t* s_bar, int* s_ok)
{
    if constexpr (!CLUSTER) {
        return true;
    } else {
        const int tid = threadIdx.x;
        const uint32_t rank = cluster_rank();
        const uint32_t bar_a = static_cast<uint32_t>(__cvta_generic_to_shared(s_bar));
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(PTabHalf) : "memory");
            const char* src = reinterpret_cast<const char*>(tab) + static_cast<size_t>(rank) * PTabHalf;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(s_tab_addr + i * 32768), "l"(src + i * 32768), "r"(32768), "r"(bar_a) : "memory");
        }
        __syncthreads();
        bool mine = false;
        for (int i = 0; i < (1 << 20) && !mine; ++i) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(bar_a) : "memory");
            mine = done != 0;
        }
        mine = __syncthreads_and(mine);
        if (tid == 0) *s_ok = mine ? 1 : 0;
        cluster_sync_all();
        const int peer_ok = ld_cluster_s32(map_to_rank(static_cast<uint32_t>(__cvta_generic_to_shared(s_ok)), rank ^ 1u));
        const bool ok = mine && peer_ok != 0;
        if (!ok && tid == 0) atomicExch(&g_pair_status, 1);
        return ok;
    }
}

// ---- staging ------------------------------------------------------------------------------------------------------
struct QuadPart {
    float4 c[4];            // c[t]: entries x = l, l+32, l+64, l+96 (+ 128 h) of the column of channel q + 8 t
};

// Warp p builds half h = p >> 3 of quad row q = p & 7.  `wstep` holds the k-step's 32 weight indices, quad row by
// quad row (the four of a quad row in one word).
template <bool CLUSTER>
__device__ __forceinline__ void fetch_part(const float* tab, uint32_t s_tab_addr, const uint8_t* wstep, int warp, int lane, QuadPart& v)
{
    const int q = warp & 7, h = warp >> 3;
    const uint32_t w4 = reinterpret_cast<const uint32_t*>(wstep)[q];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const uint32_t wi = (w4 >> (8 * t)) & 0xffu;
        if constexpr (CLUSTER) {
            const uint32_t local = s_tab_addr + (wi & 127u) * 1024u + h * 512u + lane * 16u;
            v.c[t] = ld_cluster_f4(map_to_rank(local, wi >> 7));
        } else {
            v.c[t] = __ldg(reinterpret_cast<const float4*>(tab + (wi << 8) + (h << 7)) + lane);
        }
    }
}

__device__ __forceinline__ void store_part(uint8_t* stage, int warp, int lane, const QuadPart& v)
{
    const int q = warp & 7, h = warp >> 3;
    float4* dst = reinterpret_cast<float4*>(stage + q * PPitch) + h * 128 + lane;
    dst[0] = make_float4(v.c[0].x, v.c[1].x, v.c[2].x, v.c[3].x);
    dst[32] = make_float4(v.c[0].y, v.c[1].y, v.c[2].y, v.c[3].y);
    dst[64] = make_float4(v.c[0].z, v.c[1].z, v.c[2].z, v.c[3].z);
    dst[96] = make_float4(v.c[0].w, v.c[1].w, v.c[2].w, v.c[3].w);
}

// position of channel c (0..31 within the tile) in a k-step's row of staged weight indices
__device__ __forceinline__ int p_slot(int c) { return ((c & 7) << 2) + (c >> 3); }

// ---- operand tiles ------------------------------------------------------------------------------------------------
struct PRow {
    const uint8_t* base;     // column mode: &x[n, 0, l]; image mode: &x[n, 0, 0, 0]
    int ih0, iw0;
    long long n;
    int l;
};

__device__ __forceinline__ PRow make_row(const PairArgs& a, long long r)
{
    PRow p;
    if (a.image_mode) {
        const long long hw = static_cast<long long>(a.g.OH) * a.g.OW;
        p.n = r / hw;
        p.l = static_cast<int>(r - p.n * hw);
        const int oh = p.l / a.g.OW, ow = p.l - oh * a.g.OW;
        p.base = a.x + p.n * a.g.C * a.g.H * a.g.W;
        p.ih0 = oh * a.g.SH - a.g.PH;
        p.iw0 = ow * a.g.SW - a.g.PW;
    } else {
        p.n = r / a.L;
        p.l = static_cast<int>(r - p.n * a.L);
        p.base = a.x + p.n * a.K * a.L + p.l;
        p.ih0 = p.iw0 = 0;
    }
    return p;
}

// 16 k-steps of one pixel row (thread t < rows loads row r0 + t) and of one channel (threads t < 32)
__device__ __forceinline__ void p_load_chunk(const PairArgs& a, const PRow& rc, const uint8_t* wcol, int k0, int tid,
                                             uint32_t (&xr)[4], uint32_t (&wr)[4])
{
    xr[0] = xr[1] = xr[2] = xr[3] = 0u;
    if (a.image_mode) {
        const int khw = a.g.KH * a.g.KW;
        int c = k0 / khw;
        const int rem = k0 - c * khw;
        int i = rem / a.g.KW;
        int j = rem - i * a.g.KW;
#pragma unroll
        for (int kk = 0; kk < PChunk; ++kk) {
            const int ih = rc.ih0 + i * a.g.DH;
            const int iw = rc.iw0 + j * a.g.DW;
            const bool inside = static_cast<unsigned>(ih) < static_cast<unsigned>(a.g.H) &&
                                static_cast<unsigned>(iw) < static_cast<unsigned>(a.g.W) && (k0 + kk < a.K);
            const long long off = inside ? (static_cast<long long>(c) * a.g.H + ih) * a.g.W + iw : 0LL;
            const uint32_t b = static_cast<uint32_t>(__ldg(rc.base + off)) ^ static_cast<uint32_t>(a.x_xor);
            xr[kk >> 2] |= (inside ? b : static_cast<uint32_t>(a.pad_index)) << (8 * (kk & 3));
            const bool wrap_j = ++j == a.g.KW;
            j = wrap_j ? 0 : j;
            i += wrap_j ? 1 : 0;
            const bool wrap_i = i == a.g.KH;
            i = wrap_i ? 0 : i;
            c += wrap_i ? 1 : 0;
        }
    } else {
#pragma unroll
        for (int kk = 0; kk < PChunk; ++kk) {
            if (k0 + kk < a.K) {
                const uint32_t v = static_cast<uint32_t>(__ldg(rc.base + static_cast<long long>(k0 + kk) * a.L)) ^
                                   static_cast<uint32_t>(a.x_xor);
                xr[kk >> 2] |= v << (8 * (kk & 3));
            }
        }
    }
    if (tid < PS) {
        wr[0] = wr[1] = wr[2] = wr[3] = 0u;
#pragma unroll
        for (int kk = 0; kk < PChunk; ++kk) {
            if (k0 + kk < a.K) {
                const uint32_t v = __ldg(wcol + k0 + kk);
                wr[kk >> 2] |= v << (8 * (kk & 3));
            }
        }
    }
}

__device__ __forceinline__ void p_store_chunk(uint8_t* s_x, uint8_t* s_w, int buf, int tid,
                                              const uint32_t (&xr)[4], const uint32_t (&wr)[4])
{
    uint8_t* xd = s_x + buf * PChunk * PQ + tid;
#pragma unroll
    for (int kk = 0; kk < PChunk; ++kk) xd[kk * PQ] = static_cast<uint8_t>(xr[kk >> 2] >> (8 * (kk & 3)));
    if (tid < PS) {
        uint8_t* wd = s_w + buf * PChunk * PS + p_slot(tid);
#pragma unroll
        for (int kk = 0; kk < PChunk; ++kk) wd[kk * PS] = static_cast<uint8_t>(wr[kk >> 2] >> (8 * (kk & 3)));
    }
}

// dY of the thread's 8 pixel rows x 4 channels (zero outside the problem)
__device__ __forceinline__ void load_dy(const PairArgs& a, long long r0, int c0, int warp, int lane, float (&d)[8][4])
{
    const int g = lane >> 3, q = lane & 7;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const long long r = r0 + warp * 32 + g * 8 + j;
        const long long n = r / a.L;
        const long long l = r - n * a.L;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int o = c0 + q + 8 * t;
            d[j][t] = (r < a.R && o < a.O) ? __ldg(a.dy + (n * a.O + o) * a.L + l) : 0.0f;
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------------------------------------
// GRAD_W: units are (channel tile, row tile, k-chunk), k-chunk fastest; a run keeps the dY registers of its (channel
// tile, row tile) while it walks k.  Otherwise (grad_x): units are (row tile, k-chunk); the block passes over all
// channel tiles for its run of k-chunks.
template <bool GRAD_W, bool CLUSTER>
__global__ void __launch_bounds__(PThreads, 1) pair_grad_kernel(const PairArgs a)
{
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ int s_ok;
    uint8_t* s_stage = smem + PSmemStage;
    uint8_t* s_x = smem + PSmemX;
    uint8_t* s_w = smem + PSmemW;
    float* s_red = reinterpret_cast<float*>(smem + PSmemRed);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 3, q = lane & 7;
    const uint32_t s_tab_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

    const bool ok = table_half_load<CLUSTER>(a.tab, s_tab_addr, &s_bar, &s_ok);

    long long u = static_cast<long long>(blockIdx.x) * a.units_per_cta;
    const long long u_end = min(a.total_units, u + a.units_per_cta);
    while (ok && u < u_end) {
        // ---- this segment: a (channel tile, row tile) pair and a range of k-chunks
        int ct, rt, ch_beg, ch_end;
        if (GRAD_W) {
            const long long pair = u / a.nchunks;
            ch_beg = static_cast<int>(u - pair * a.nchunks);
            ch_end = static_cast<int>(min(static_cast<long long>(a.nchunks), ch_beg + (u_end - u)));
            ct = static_cast<int>(pair / a.row_tiles);
            rt = static_cast<int>(pair - static_cast<long long>(ct) * a.row_tiles);
        } else {
            rt = static_cast<int>(u / a.nchunks);
            ch_beg = static_cast<int>(u - static_cast<long long>(rt) * a.nchunks);
            ch_end = static_cast<int>(min(static_cast<long long>(a.nchunks), ch_beg + (u_end - u)));
            ct = 0;
        }
        const long long r0 = static_cast<long long>(rt) * PQ;
        const PRow rc = make_row(a, min(r0 + tid, a.R - 1));
        const int n_ct = GRAD_W ? 1 : a.ch_tiles;
        for (int pass = 0; pass < n_ct; ++pass, ++ct) {
            const int c0 = ct * PS;
            const uint8_t* wcol = a.w + static_cast<long long>(min(c0 + tid, a.O - 1)) * a.K;
            float d[8][4];
            load_dy(a, r0, c0, warp, lane, d);
            uint32_t xr[4], wr[4];
            __syncthreads();                              // previous pass / segment is done with the tiles
            p_load_chunk(a, rc, wcol, ch_beg * PChunk, tid, xr, wr);
            p_store_chunk(s_x, s_w, 0, tid, xr, wr);
            __syncthreads();
            {
                QuadPart v;
                fetch_part<CLUSTER>(a.tab, s_tab_addr, s_w, warp, lane, v);
                store_part(s_stage, warp, lane, v);
            }
            __syncthreads();
            int step = 0;
            const int kend = min(a.K, ch_end * PChunk);
            for (int ci = ch_beg; ci < ch_end; ++ci) {
                const int k0 = ci * PChunk;
                const int kc = min(PChunk, kend - k0);
                const int cur = (ci - ch_beg) & 1;
                const bool has_next = ci + 1 < ch_end;
                if (has_next) p_load_chunk(a, rc, wcol, k0 + PChunk, tid, xr, wr);
                for (int kk = 0; kk < kc; ++kk, ++step) {
                    if (has_next && kk == 4) p_store_chunk(s_x, s_w, cur ^ 1, tid, xr, wr);
                    const uint8_t* xrow = s_x + (cur * PChunk + kk) * PQ + warp * 32 + g * 8;
                    const uint8_t* wstep = s_w + (cur * PChunk + kk) * PS;
                    const uint8_t* wnext = nullptr;
                    if (kk + 1 < kc) wnext = wstep + PS;
                    else if (has_next) wnext = s_w + ((cur ^ 1) * PChunk) * PS;
                    const uint8_t* stage_cur = s_stage + (step & 1) * PStageBytes;
                    QuadPart v;
                    if (wnext != nullptr) fetch_part<CLUSTER>(a.tab, s_tab_addr, wnext, warp, lane, v);

                    const uint2 xb = *reinterpret_cast<const uint2*>(xrow);          // the 8 rows' activation indices
                    const float4* col = reinterpret_cast<const float4*>(stage_cur + q * PPitch);
                    const int k = k0 + kk;
                    if (GRAD_W) {
                        float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t xi = ((j < 4 ? xb.x : xb.y) >> (8 * (j & 3))) & 0xffu;
                            const float4 e = col[xi];
                            p0 = fmaf(d[j][0], e.x, p0); p1 = fmaf(d[j][1], e.y, p1);
                            p2 = fmaf(d[j][2], e.z, p2); p3 = fmaf(d[j][3], e.w, p3);
                        }
                        // transposing reduction over the four row groups (lane bits 3 and 4): lane c ends with channel c
                        const bool hi = (g & 2) != 0, odd = (g & 1) != 0;
                        const float k0v = (hi ? p2 : p0) + __shfl_xor_sync(0xffffffffu, hi ? p0 : p2, 16);
                        const float k1v = (hi ? p3 : p1) + __shfl_xor_sync(0xffffffffu, hi ? p1 : p3, 16);
                        const float val = (odd ? k1v : k0v) + __shfl_xor_sync(0xffffffffu, odd ? k0v : k1v, 8);
                        s_red[((step & 1) * 16 + warp) * PS + lane] = val;
                    } else {
                        float p[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t xi = ((j < 4 ? xb.x : xb.y) >> (8 * (j & 3))) & 0xffu;
                            const float4 e = col[xi];
                            p[j] = fmaf(d[j][0], e.x, fmaf(d[j][1], e.y, fmaf(d[j][2], e.z, d[j][3] * e.w)));
                        }
                        // transposing reduction over the eight quad rows (lane bits 0..2): lane r ends with pixel row r
                        const bool b2 = (q & 4) != 0, b1 = (q & 2) != 0, b0 = (q & 1) != 0;
                        float a4[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            a4[i] = (b2 ? p[4 + i] : p[i]) + __shfl_xor_sync(0xffffffffu, b2 ? p[i] : p[4 + i], 4);
                        float a2[2];
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            a2[i] = (b1 ? a4[2 + i] : a4[i]) + __shfl_xor_sync(0xffffffffu, b1 ? a4[i] : a4[2 + i], 2);
                        const float val = (b0 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, b0 ? a2[0] : a2[1], 1);
                        const long long r = r0 + warp * 32 + lane;
                        if (r < a.R) {
                            if (a.image_mode) {
                                // the tap (c, i, j) of output pixel r: add to the image pixel it read (padded taps: nowhere)
                                const int khw = a.g.KH * a.g.KW;
                                const int c = k / khw;
                                const int rem = k - c * khw;
                                const int ti = rem / a.g.KW, tj = rem - ti * a.g.KW;
                                const long long hw = static_cast<long long>(a.g.OH) * a.g.OW;
                                const long long n = r / hw;
                                const int l = static_cast<int>(r - n * hw);
                                const int oh = l / a.g.OW, ow = l - oh * a.g.OW;
                                const int ih = oh * a.g.SH - a.g.PH + ti * a.g.DH;
                                const int iw = ow * a.g.SW - a.g.PW + tj * a.g.DW;
                                if (static_cast<unsigned>(ih) < static_cast<unsigned>(a.g.H) &&
                                    static_cast<unsigned>(iw) < static_cast<unsigned>(a.g.W))
                                    atomicAdd(a.out + ((n * a.g.C + c) * a.g.H + ih) * a.g.W + iw, val);
                            } else {
                                const long long n = r / a.L;
                                const long long l = r - n * a.L;
                                float* dst = a.out + (n * a.K + k) * a.L + l;
                                *dst = pass == 0 ? val : *dst + val;
                            }
                        }
                    }
                    if (wnext != nullptr) store_part(s_stage + ((step + 1) & 1) * PStageBytes, warp, lane, v);
                    __syncthreads();
                    if (GRAD_W && warp == 0) {
                        // the k-step's 32 channel sums over this block's 512 rows (drained while the next step runs)
                        float s = 0.0f;
#pragma unroll
                        for (int w16 = 0; w16 < 16; ++w16) s += s_red[((step & 1) * 16 + w16) * PS + lane];
                        const int o = c0 + lane;
                        if (o < a.O) atomicAdd(a.out + static_cast<long long>(o) * a.K + k, s);
                    }
                }
            }
        }
        u += ch_end - ch_beg;
    }
    if constexpr (CLUSTER) cluster_sync_all();       // the peer may still be reading this block's half of the table
}

// ---- forward on a table of the fp32 class ----------------------------------------------------------------------------
// y[r, o] = sum_k T[w(o,k)][x(r,k)] accumulated in fp32 in ascending k (the reference's order,
// approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:278-281, 344-359; it gathers from the 256 KB table in global
// memory).  Tiles of 512 pixel rows x 32 channels, the whole reduction inside one block (no cut along k, so the sum
// order is exactly ascending k), tiles dealt round-robin to a persistent grid, column tile fastest.
struct FwdEpilogue {
    float* y;
    const float* alpha;
    const float* beta;
    const float* zero_x;
    const float* zero_w;
    const int* wsum;
};

__device__ __forceinline__ float fwd_finalize(float total, int xsum, int o, int K, const FwdEpilogue& ep)
{
    float v = total;
    if (ep.zero_x != nullptr) {
        // integer zero-point terms added in double, one rounding back to fp32
        const long long zx = llrintf(__ldg(ep.zero_x));
        const long long zw = llrintf(__ldg(ep.zero_w + o));
        const long long ws = __ldg(ep.wsum + o);
        v = static_cast<float>(static_cast<double>(total) +
                               static_cast<double>(-zw * xsum - zx * ws + static_cast<long long>(K) * zx * zw));
    }
    // unfused, like every epilogue of the LUT GEMM (two roundings: the reference multiplies and adds separately)
    if (ep.alpha != nullptr) v = __fmul_rn(v, __ldg(ep.alpha + o));
    if (ep.beta != nullptr) v = __fadd_rn(v, __ldg(ep.beta + o));
    return v;
}

template <bool CLUSTER>
__global__ void __launch_bounds__(PThreads, 1) pair_fwd_kernel(PairArgs a, const FwdEpilogue ep)
{
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ int s_ok;
    uint8_t* s_stage = smem + PSmemStage;
    uint8_t* s_x = smem + PSmemX;
    uint8_t* s_w = smem + PSmemW;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 3, q = lane & 7;
    const uint32_t s_tab_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const bool ok = table_half_load<CLUSTER>(a.tab, s_tab_addr, &s_bar, &s_ok);
    if (a.pad_index < 0) a.pad_index = min(255, max(0, static_cast<int>(llrintf(__ldg(ep.zero_x)))));
    const bool want_xsum = ep.zero_x != nullptr;
    const long long tiles = static_cast<long long>(a.row_tiles) * a.ch_tiles;
    for (long long tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
        const int rt = static_cast<int>(tile / a.ch_tiles);
        const int c0 = static_cast<int>(tile - static_cast<long long>(rt) * a.ch_tiles) * PS;
        const long long r0 = static_cast<long long>(rt) * PQ;
        const PRow rc = make_row(a, min(r0 + tid, a.R - 1));
        const uint8_t* wcol = a.w + static_cast<long long>(min(c0 + tid, a.O - 1)) * a.K;
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) { acc[j][0] = 0.0f; acc[j][1] = 0.0f; acc[j][2] = 0.0f; acc[j][3] = 0.0f; }
        int xsum = 0;
        uint32_t xr[4], wr[4];
        __syncthreads();                                  // the previous tile is done with the tiles and the turning space
        p_load_chunk(a, rc, wcol, 0, tid, xr, wr);
        p_store_chunk(s_x, s_w, 0, tid, xr, wr);
        __syncthreads();
        {
            QuadPart v;
            fetch_part<CLUSTER>(a.tab, s_tab_addr, s_w, warp, lane, v);
            store_part(s_stage, warp, lane, v);
        }
        __syncthreads();
        int step = 0;
        for (int ci = 0; ci < a.nchunks; ++ci) {
            const int k0 = ci * PChunk;
            const int kc = min(PChunk, a.K - k0);
            const int cur = ci & 1;
            const bool has_next = ci + 1 < a.nchunks;
            if (has_next) p_load_chunk(a, rc, wcol, k0 + PChunk, tid, xr, wr);
            for (int kk = 0; kk < kc; ++kk, ++step) {
                if (has_next && kk == 4) p_store_chunk(s_x, s_w, cur ^ 1, tid, xr, wr);
                const uint8_t* xrow_w = s_x + (cur * PChunk + kk) * PQ + warp * 32;
                const uint8_t* wstep = s_w + (cur * PChunk + kk) * PS;
                const uint8_t* wnext = nullptr;
                if (kk + 1 < kc) wnext = wstep + PS;
                else if (has_next) wnext = s_w + ((cur ^ 1) * PChunk) * PS;
                QuadPart v;
                if (wnext != nullptr) fetch_part<CLUSTER>(a.tab, s_tab_addr, wnext, warp, lane, v);
                if (want_xsum) xsum += static_cast<int>(xrow_w[lane]);
                const uint2 xb = *reinterpret_cast<const uint2*>(xrow_w + g * 8);
                const float4* col = reinterpret_cast<const float4*>(s_stage + (step & 1) * PStageBytes + q * PPitch);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t xi = ((j < 4 ? xb.x : xb.y) >> (8 * (j & 3))) & 0xffu;
                    const float4 e = col[xi];
                    acc[j][0] += e.x; acc[j][1] += e.y; acc[j][2] += e.z; acc[j][3] += e.w;
                }
                if (wnext != nullptr) store_part(s_stage + ((step + 1) & 1) * PStageBytes, warp, lane, v);
                __syncthreads();
            }
        }
        // ---- epilogue: thread (g, q) holds rows warp*32 + g*8 + j, channels c0 + q + 8 t
        if (a.L == 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const long long r = r0 + warp * 32 + g * 8 + j;
                const int xs = __shfl_sync(0xffffffffu, xsum, g * 8 + j);
                if (r >= a.R) continue;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int o = c0 + q + 8 * t;
                    if (o < a.O) ep.y[r * a.O + o] = fwd_finalize(acc[j][t], xs, o, a.K, ep);
                }
            }
        } else {
            // the fast axis of y[n, o, l] is the pixel: turn the warp's 32 x 32 tile around in the (now free) stage area
            constexpr int kPitch = 33;
            float* turn = reinterpret_cast<float*>(s_stage) + warp * (32 * kPitch);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int xs = __shfl_sync(0xffffffffu, xsum, g * 8 + j);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int oc = q + 8 * t;
                    turn[oc * kPitch + g * 8 + j] = (c0 + oc < a.O) ? fwd_finalize(acc[j][t], xs, c0 + oc, a.K, ep) : 0.0f;
                }
            }
            __syncwarp();
            const long long r = r0 + warp * 32 + lane;
            if (r < a.R) {
                const long long n = r / a.L;
                const long long l = r - n * a.L;
                float* dst = ep.y + (n * a.O + c0) * a.L + l;
                const int ncols = min(PS, a.O - c0);
                for (int c = 0; c < ncols; ++c) dst[static_cast<long long>(c) * a.L] = turn[c * kPitch + lane];
            }
        }
    }
    if constexpr (CLUSTER) cluster_sync_all();       // the peer may still be reading this block's half of the table
}

template <bool GRAD_W, bool CLUSTER>
static int launch_pair(const PairArgs& a, int ctas, cudaStream_t stream)
{
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return ATB_ERR_CUDA;
    }
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(pair_grad_kernel<GRAD_W, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, PSmemTotal);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(PThreads);
    cfg.dynamicSmemBytes = PSmemTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CLUSTER ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, pair_grad_kernel<GRAD_W, CLUSTER>, a);
    if (e != cudaSuccess) { set_error("pair_grad_kernel launch: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    return check_launch("pair_grad_kernel");
}

template <bool CLUSTER>
static int launch_pair_fwd(const PairArgs& a, const FwdEpilogue& ep, int ctas, cudaStream_t stream)
{
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return ATB_ERR_CUDA;
    }
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(pair_fwd_kernel<CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, PSmemTotal);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(PThreads);
    cfg.dynamicSmemBytes = PSmemTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CLUSTER ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, pair_fwd_kernel<CLUSTER>, a, ep);
    if (e != cudaSuccess) { set_error("pair_fwd_kernel launch: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    return check_launch("pair_fwd_kernel");
}

int pair_forward_launch(const PairFwdParams& p, int mode, cudaStream_t stream)
{
    PairArgs a{};
    a.x = p.x; a.w = p.w; a.tab = p.tab;
    a.R = p.R; a.K = p.K; a.L = p.L; a.O = p.O;
    a.image_mode = p.image_mode; a.x_xor = p.x_xor; a.pad_index = p.pad_index; a.g = p.g;
    a.row_tiles = ceil_div(a.R, PQ);
    a.ch_tiles = ceil_div(a.O, PS);
    a.nchunks = ceil_div(a.K, PChunk);
    const FwdEpilogue ep{p.y, p.alpha, p.beta, p.zero_x, p.zero_w, p.wsum};
    const bool cluster = (mode & 1) == 0;
    const long long tiles = static_cast<long long>(a.row_tiles) * a.ch_tiles;
    int sms = sm_count();
    if (cluster) sms &= ~1;
    long long ctas = tiles < sms ? tiles : sms;
    if (cluster && (ctas & 1)) ++ctas;
    return cluster ? launch_pair_fwd<true>(a, ep, static_cast<int>(ctas), stream)
                   : launch_pair_fwd<false>(a, ep, static_cast<int>(ctas), stream);
}

__global__ void pair_zero_kernel(float* p, long long n)
{
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = 0.0f;
}

// mode bit 0: 0 = table halves in a two-block cluster's shared memory, 1 = staging reads from global memory
static int run_pair(PairArgs a, bool grad_w, int mode, cudaStream_t stream)
{
    a.row_tiles = ceil_div(a.R, PQ);
    a.ch_tiles = ceil_div(a.O, PS);
    a.nchunks = ceil_div(a.K, PChunk);
    a.total_units = grad_w ? static_cast<long long>(a.ch_tiles) * a.row_tiles * a.nchunks
                           : static_cast<long long>(a.row_tiles) * a.nchunks;
    const bool cluster = (mode & 1) == 0;
    int sms = sm_count();
    if (cluster) sms &= ~1;
    long long ctas = a.total_units < sms ? a.total_units : sms;
    const long long units = (a.total_units + ctas - 1) / ctas;
    ctas = (a.total_units + units - 1) / units;
    if (cluster && (ctas & 1)) ++ctas;                 // a block without work still holds its half of the table
    ATB_REQUIRE(units <= 2147483647LL, "run too long");
    a.units_per_cta = static_cast<int>(units);
    if (grad_w) return cluster ? launch_pair<true, true>(a, static_cast<int>(ctas), stream) : launch_pair<true, false>(a, static_cast<int>(ctas), stream);
    return cluster ? launch_pair<false, true>(a, static_cast<int>(ctas), stream) : launch_pair<false, false>(a, static_cast<int>(ctas), stream);
}

}  // namespace atb

using namespace atb;

extern "C" int atb_pair_status(int* status /*host*/)
{
    ATB_REQUIRE(status != nullptr, "status is null");
    cudaError_t e = cudaMemcpyFromSymbol(status, g_pair_status, sizeof(int));
    if (e != cudaSuccess) { set_error("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e)); return ATB_ERR_CUDA; }
    return ATB_OK;
}

extern "C" size_t atb_pair_table_bytes(void) { return 65536 * sizeof(float); }

extern "C" int atb_pair_table_prepare(const float* table, float* prepared, void* stream)
{
    ATB_REQUIRE(table != nullptr && prepared != nullptr, "null pointer");
    ATB_REQUIRE(aligned_to(prepared, 16), "prepared table must be 16-byte aligned");
    pair_table_prepare_kernel<<<256, 256, 0, static_cast<cudaStream_t>(stream)>>>(table, prepared);
    return check_launch("pair_table_prepare_kernel");
}

extern "C" int atb_custom_bwd_dx(const uint8_t* x, const uint8_t* w, const float* dy, const float* dx_prepared,
                                 float* grad_x, int N, int K, int L, int O, int mode, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    const long long R = static_cast<long long>(N) * L;
    if (R * K == 0) return ATB_OK;
    ATB_REQUIRE(x && grad_x && dx_prepared && (O == 0 || (w && dy)), "null pointer");
    ATB_REQUIRE(R <= 2147483647LL, "N*L too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (O == 0) {
        pair_zero_kernel<<<grid_for(R * K, 256, 4096), 256, 0, s>>>(grad_x, R * K);
        return check_launch("pair_zero_kernel");
    }
    PairArgs a{};
    a.x = x; a.w = w; a.dy = dy; a.tab = dx_prepared; a.out = grad_x;
    a.R = R; a.K = K; a.L = L; a.O = O;
    return run_pair(a, false, mode, s);
}

extern "C" int atb_custom_bwd_dw(const uint8_t* x, const uint8_t* w, const float* dy, const float* dw_prepared,
                                 float* grad_w, int N, int K, int L, int O, int mode, void* stream)
{
    ATB_REQUIRE(N >= 0 && K >= 0 && L >= 0 && O >= 0, "negative dimension");
    if (static_cast<long long>(O) * K == 0) return ATB_OK;
    const long long R = static_cast<long long>(N) * L;
    ATB_REQUIRE(w && grad_w && dw_prepared && (R == 0 || (x && dy)), "null pointer");
    ATB_REQUIRE(R <= 2147483647LL, "N*L too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    pair_zero_kernel<<<grid_for(static_cast<long long>(O) * K, 256, 4096), 256, 0, s>>>(grad_w, static_cast<long long>(O) * K);
    int rc = check_launch("pair_zero_kernel");
    if (rc != ATB_OK || R == 0) return rc;
    PairArgs a{};
    a.x = x; a.w = w; a.dy = dy; a.tab = dw_prepared; a.out = grad_w;
    a.R = R; a.K = K; a.L = L; a.O = O;
    return run_pair(a, true, mode, s);
}

// Image form: x is the quantised image (int8 values or uint8 indices), taps outside it look up `pad_index`;
// grad_x is the gradient with respect to the image (the fold is done in the kernel), grad_w is [O, C*kh*kw].
extern "C" int atb_custom_conv_bwd(const void* x, int dtype, const uint8_t* w, const float* dy,
                                   const float* dx_prepared, const float* dw_prepared, float* grad_x, float* grad_w,
                                   int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw, int ph, int pw,
                                   int dh, int dw_, int pad_index, int mode, void* stream)
{
    ATB_REQUIRE(N >= 0 && C >= 0 && H >= 0 && W >= 0 && O >= 0, "negative dimension");
    ATB_REQUIRE(dtype == ATB_I8 || dtype == ATB_U8, "image must be int8 values or uint8 indices");
    ATB_REQUIRE(pad_index >= 0 && pad_index <= 255, "pad_index out of range");
    int OH = 0, OW = 0;
    ATB_REQUIRE(conv_out_shape(H, W, kh, kw, sh, sw, ph, pw, dh, dw_, &OH, &OW), "conv geometry yields empty output");
    const long long K = static_cast<long long>(C) * kh * kw;
    const long long R = static_cast<long long>(N) * OH * OW;
    ATB_REQUIRE(K <= 2147483647LL && R <= 2147483647LL, "dimensions too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PairArgs a{};
    a.x = static_cast<const uint8_t*>(x); a.w = w; a.dy = dy;
    a.R = R; a.K = static_cast<int>(K); a.L = OH * OW; a.O = O;
    a.image_mode = 1; a.x_xor = dtype == ATB_I8 ? 0x80 : 0; a.pad_index = pad_index;
    a.g = ConvGeom{C, H, W, kh, kw, sh, sw, ph, pw, dh, dw_, OH, OW};
    int rc = ATB_OK;
    if (grad_x != nullptr && static_cast<long long>(N) * C * H * W > 0) {
        const long long numel = static_cast<long long>(N) * C * H * W;
        pair_zero_kernel<<<grid_for(numel, 256, 4096), 256, 0, s>>>(grad_x, numel);
        rc = check_launch("pair_zero_kernel");
        if (rc != ATB_OK) return rc;
        if (R * K * O > 0) {
            ATB_REQUIRE(x && w && dy && dx_prepared, "null pointer");
            a.tab = dx_prepared; a.out = grad_x;
            rc = run_pair(a, false, mode, s);
            if (rc != ATB_OK) return rc;
        }
    }
    if (grad_w != nullptr && O * K > 0) {
        pair_zero_kernel<<<grid_for(O * K, 256, 4096), 256, 0, s>>>(grad_w, O * K);
        rc = check_launch("pair_zero_kernel");
        if (rc != ATB_OK) return rc;
        if (R > 0) {
            ATB_REQUIRE(x && w && dy && dw_prepared, "null pointer");
            a.tab = dw_prepared; a.out = grad_w;
            rc = run_pair(a, true, mode, s);
        }
    }
    return rc;
}
