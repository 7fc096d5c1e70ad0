/* C ABI of libapproxtorch_b200.so — the drop-in boundary of the approximate-multiplier hot path.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless a comment says
 * "host"; `stream` is a cudaStream_t passed as void*.  Every entry point enqueues work on
 * `stream` and returns without synchronising.  Return value: 0 = success, otherwise one of
 * the ATB_ERR_* codes; atb_last_error() gives the message of the calling thread's last
 * failure.  No entry point allocates device memory unless its comment says so: outputs and
 * scratch buffers are supplied by the caller (the Python binding uses torch tensors).
 *
 * Each declaration names the reference interface it replaces; paths are relative to the
 * reference project root.
 *
 * Shape letters: N batch, K = C*kh*kw reduction, L = OH*OW output pixels, O output channels,
 * R = N*L pixel rows.  LUT index rule: table row = activation index, column = weight index,
 * flat = idx(x)*256 + idx(w); idx_int8(v) = v+128, idx_uint8(v) = v.
 */
#ifndef APPROXTORCH_B200_H
#define APPROXTORCH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATB_OK 0
#define ATB_ERR_INVALID 1   /* bad argument (shape, null pointer, unsupported size) */
#define ATB_ERR_CUDA 2      /* a CUDA runtime call or launch failed */
#define ATB_ERR_SCRATCH 3   /* caller-supplied scratch buffer too small */

/* element types accepted where an operand may be fp32 integer values, int8 values or uint8 LUT indices
 * (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:69-80, 353-355) */
#define ATB_F32 0
#define ATB_I8 1
#define ATB_U8 2

const char* atb_last_error(void);
int atb_version(void);
/* Device-side error word of the current device (host pointer out; synchronises).  0 = none; 1 = a LUT GEMM block
 * gave up waiting for its table copy and left its tiles unwritten; 2 = atb_lut_conv2d_rows_fwd was given a table of
 * the fp32 class and wrote nothing.  (No counterpart in the reference.) */
int atb_device_status(int* status /*host*/);

/* ---- LUT image --------------------------------------------------------------------------
 * Device-side image of a 256x256 fp32 table: 16-bit and fp32 copies, natural and transposed,
 * plus two validity flags the kernels branch on (int16-exact, uint16-exact).  Replaces
 * prepare_lut_kernel and the per-call allocations around it
 * (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:116-142,
 *  approxtorch/backend/csrc/claude/bgemm_float_claude.cu:163-192); built once per table, not per call. */
size_t atb_lut_image_bytes(void);
int atb_lut_prepare(const float* lut /*[65536]*/, void* image /*atb_lut_image_bytes()*/, void* stream);
/* Class of a prepared table, read back to the host (synchronises `stream`): 0 = int16-exact, 1 = uint16-exact,
 * 2 = neither (fp32).  The eligibility rules are the reference's
 * (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:126-134).  A host that knows the class is 2 can ask for
 * the kernel that keeps the fp32 table on chip (cfg bit 24 of the GEMM / conv entries). */
int atb_lut_image_class(const void* lut_image, int* cls /*host*/, void* stream);

/* ---- operand prepasses ------------------------------------------------------------------ */
/* fp32 integer-valued operand -> uint8 LUT index, clamp(rn(v)+offset, 0, 255)
 * (quantize_to_u8_kernel, approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:62-97). */
int atb_quantize_u8(const float* in, uint8_t* out, long long numel, int offset, void* stream);
/* B[K,N] with arbitrary element strides (fp32 values or uint8 indices) -> uint8 [N,K]
 * (quantize_transpose_u8_kernel, approxtorch/backend/csrc/claude/gemm.cu:68-95). */
int atb_quantize_transpose_u8(const void* b, int dtype, int K, int N, long long stride_k,
                              long long stride_n, int offset, uint8_t* out, void* stream);
/* quantised image [N,C,H,W] (fp32 / int8 / uint8) -> uint8 LUT-index columns [N, C*kh*kw, OH*OW];
 * taps outside the image get `pad_index` (128 = quantised zero of the signed path)
 * (im2col_u8, approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:216-269, 737-791). */
int atb_im2col_u8(const void* x, int dtype, int N, int C, int H, int W, int kh, int kw, int sh, int sw,
                  int ph, int pw, int dh, int dw, int pad_index, uint8_t* out, void* stream);

/* ---- LUT GEMM / conv forward --------------------------------------------------------------
 * y[n,o,l] = alpha[o] * t + beta[o],
 * t = sum_k lut[x_idx][w_idx] - zw[o]*xsum[n,l] - zx*wsum[o] + K*zx*zw[o]
 * alpha/beta are optional (NULL = 1 / 0).  The zero-point terms are formed only when zero_x != NULL:
 * zx = *zero_x and zw = zero_w[o] are integer-valued fp32, wsum[o] = sum_k w_idx[o,k] (int32),
 * xsum = sum_k x_idx of the row; they are combined in integer arithmetic before the single
 * conversion to fp32.  Integer tables accumulate in int32 (exact; K up to 65536), other tables in fp32 in
 * ascending k (ascending k inside a k-segment, segments added in ascending order when a tile is cut).
 *
 * Scheduling: the work is cut into units of (64-channel tile, 16-step k-chunk) and dealt out in equal contiguous
 * runs, one per thread block (persistent stream-K).  A tile that lies inside one run is written straight to y; a
 * tile cut between runs is finished by the last of its blocks to arrive, the others having parked their partial
 * sums in `scratch` (no reduction kernel, nobody waits).  Integer tables give the same bits under every plan.
 *
 * cfg: -1 automatic.  Otherwise bits 0-15 pixel rows per tile (a multiple of 32 up to 512; 0 = automatic) and
 * bits 16-23 the cutting rule: 0 automatic, 1 never cut a tile (runs of whole tiles), S > 1 cut every tile into
 * (about) S k-segments, one block each.  Bit 24: the table is known to be of the fp32 class (atb_lut_image_class):
 * run it on the kernel that holds the 256 KB fp32 table in the shared memory of a two-block cluster, half each,
 * read across the cluster (tiles of 512 rows x 32 channels, whole reductions in ascending k, no scratch); without
 * the bit such tables are gathered from global memory.  Bit 25 (with bit 24): stage from global memory instead of
 * the cluster's shared memory.  Other bits are ignored.
 *
 * The plan says how a launch will be laid out and how much scratch (bytes) it needs. */
typedef struct {
    int block_rows;       /* pixel rows per tile: a multiple of 32 up to 512 */
    int blocks;           /* thread blocks launched (at most one per SM under the automatic plan) */
    int units_per_block;  /* (tile, k-chunk) units in a block's run */
    int chunks_per_tile;  /* ceil(K / 16) */
    int cut_tiles;        /* 1 when runs end inside tiles: needs scratch_bytes of scratch (16-byte aligned) */
    size_t scratch_bytes; /* arrival counters + two parking slots per block; 0 when no tile is cut */
} atb_gemm_plan;

int atb_lut_gemm_plan(long long R, int K, int O, int wb_rows, int cfg, atb_gemm_plan* plan /*host*/);

/* Batched LUT GEMM on uint8 index operands.  x is [N,K,L] (l fastest; L == 1 gives the torch.mm
 * layout A[M,K]); w is [O,K] shared by all rows (wb_rows == 0) or one [O,K] matrix per `wb_rows`
 * consecutive pixel rows, `w_batch_stride` bytes apart.  Replaces bgemm_forward_save_cfg_impl and
 * gemm_forward_save_cfg_impl (approxtorch/backend/csrc/claude/bgemm_float_claude.cu:70-205,
 * approxtorch/backend/csrc/claude/gemm.cu:97-232) and the dequantisation of
 * approxtorch/nn/Conv2d_int8.py:213-218 when alpha/beta are given. */
int atb_lut_bgemm_fwd(const uint8_t* x, const uint8_t* w, const void* lut_image, float* y,
                      int N, int K, int L, int O, int wb_rows, long long w_batch_stride,
                      const float* alpha, const float* beta, const float* zero_x, const float* zero_w, const int* wsum,
                      int cfg, void* scratch, size_t scratch_bytes, void* stream);

/* The same batched LUT GEMM for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its operators allocate their split-K workspace from torch's allocator on every call.)
 * A host that is capturing a CUDA graph, runs under a closed memory pool, or binds this library from a
 * runtime that cannot create device buffers inside an operator call has no scratch buffer to hand in, so
 * this variant keeps the parked partial sums of cut tiles in a fixed area of ATB_STATIC_SCRATCH_BYTES bytes of device
 * global memory that is part of the library image: every GPU that loads the library holds it until the
 * process exits.  Arguments and results are those of atb_lut_bgemm_fwd; shapes whose plan needs more
 * scratch than the area holds are refused with ATB_ERR_SCRATCH (atb_lut_gemm_plan reports the need, and
 * cfg can choose a plan that cuts no tile, or shorter tiles).  The area's device address is looked up once per device, by the first of
 * atb_static_scratch_bytes() or atb_lut_bgemm_fwd_noalloc() called while that device is current: call
 * atb_static_scratch_bytes() on every device you will use before starting any stream capture.  The
 * address is remembered per device ordinal for the life of the process (a cudaDeviceReset invalidates it;
 * do not reset a device between calls).  All calls on a device share the area and it keeps what the
 * last call left; the kernels overwrite every element they later read, so nothing has to be cleared,
 * but two such calls that overlap in time on one GPU (different streams) race on it. */
#define ATB_STATIC_SCRATCH_BYTES (32u << 20)
size_t atb_static_scratch_bytes(void);
int atb_lut_bgemm_fwd_noalloc(const uint8_t* x, const uint8_t* w, const void* lut_image, float* y,
                              int N, int K, int L, int O, int wb_rows, long long w_batch_stride,
                              const float* alpha, const float* beta, const float* zero_x, const float* zero_w, const int* wsum,
                              int cfg, void* stream);

/* im2col-free approximate Conv2d forward on the quantised image (int8 values or uint8 indices):
 * the column matrix is never materialised; taps outside the image look up `pad_index`
 * (pad_index == -1: the rounded value of *zero_x, read on the device, so no host copy is needed).
 * Replaces im2col_u8 + bgemm_fake_int8_claude_save + dequant
 * (approxtorch/nn/bgemm_int8.py:244-256, approxtorch/nn/Conv2d_int8.py:207-218) and, with zw/cterm,
 * the zero-point correction of approxtorch/nn/Conv2d_uint8.py:283-323 when zero_x is given. */
int atb_lut_conv2d_fwd(const void* x, int dtype, const uint8_t* w /*[O, C*kh*kw]*/, const void* lut_image,
                       float* y /*[N,O,OH,OW]*/, int N, int C, int H, int W, int O, int kh, int kw,
                       int sh, int sw, int ph, int pw, int dh, int dw, int pad_index,
                       const float* alpha, const float* beta, const float* zero_x, const float* zero_w, const int* wsum,
                       int cfg, void* scratch, size_t scratch_bytes, void* stream);

/* ---- the same convolution with the output channels as tile rows ----------------------------------
 * For operands with few pixel rows and many channels (late layers at small batch) the 512-row tiles of
 * atb_lut_conv2d_fwd are badly filled (784 pixels = 1.5 tiles).  Here the tile rows are the output channels and the
 * 64 tile columns are pixels: the row operand is the weight matrix w [O,K], the column operand the pixel matrix
 * pix [P,K] (P = N*L output pixels; pix[p,k] = operand index of tap k of pixel p, written by atb_pixel_rows_u8, which
 * also returns pixsum[p] = sum_k pix[p,k] for the zero-point correction), and the table image is the image of the
 * TRANSPOSED table (lut_t[a][b] = lut[b][a], prepared like any other).  Integer table classes only
 * (atb_lut_image_class; an fp32-class image raises device status 2 and writes nothing).  Same results bit for bit as
 * atb_lut_conv2d_fwd: y [N,O,L] fp32, alpha/beta/zero_w [O], zero_x scalar.  atb_lut_gemm_rows_plan gives the scratch
 * need (cfg as for atb_lut_gemm_plan).  (No counterpart in the reference: its kernels have one orientation.) */
int atb_pixel_rows_u8(const void* x, int dtype, int N, int C, int H, int W, int kh, int kw, int sh, int sw,
                      int ph, int pw, int dh, int dw, int pad_index, const float* zero_x /*scalar or NULL*/,
                      uint8_t* pix /*[N*OH*OW, C*kh*kw]*/, int* pixsum /*[N*OH*OW] or NULL*/, void* stream);
int atb_lut_gemm_rows_plan(int O, int K, long long P, int cfg, atb_gemm_plan* plan);
int atb_lut_conv2d_rows_fwd(const uint8_t* w /*[O,K]*/, const uint8_t* pix /*[P,K]*/, const void* lut_image_t, float* y,
                            int O, int K, long long P, int L,
                            const float* alpha, const float* beta, const float* zero_x,
                            const float* zero_w, const int* pixsum,
                            int cfg, void* scratch, size_t scratch_bytes, void* stream);

/* ---- fake quantisation -------------------------------------------------------------------- */
/* result[0] = max|x| (result[1] = min x, result[2] = max x when want_minmax).  `result` must hold 3 floats;
 * it is initialised by the call.  Replaces x.abs().max() / amin / amax of
 * approxtorch/nn/Conv2d_int8.py:139 and approxtorch/nn/Conv2d_uint8.py:229-230. */
int atb_absmax(const float* x, long long numel, int want_minmax, float* result, void* stream);
/* (q fp32, mask bool) = fake-quant of x with a 1-element device scale (zero_point NULL = symmetric)
 * (approxtorch/backend/csrc/claude/quantization.cu:54-110, 149-183). */
int atb_fakequant_fwd(const float* x, const float* scale, const float* zero_point, int qmin, int qmax,
                      float* q, uint8_t* mask, long long numel, void* stream);
/* gx = (mask ? go : 0) / max(scale, 1e-12) (approxtorch/backend/csrc/claude/quantization.cu:113-143). */
int atb_fakequant_bwd(const float* go, const uint8_t* mask, const float* scale, float* gx,
                      long long numel, void* stream);
/* Fused form used by the layers: same arithmetic, but writes the 1-byte quantised image (int8 value,
 * or uint8 index when zero_point != NULL) and the mask instead of an fp32 tensor; `mask` may be NULL. */
int atb_quantize_image(const float* x, const float* scale, const float* zero_point, int qmin, int qmax,
                       void* q8, uint8_t* mask, long long numel, void* stream);
/* per-output-channel weight fake-quant: w [O, inner] fp32, scale[O] (zero_point[O] or NULL) ->
 * uint8 LUT index (value + index_offset), mask, optional fp32 q and optional per-channel index sum
 * (approxtorch/nn/quantization.py:98-133). */
int atb_quantize_weight(const float* w, const float* scale, const float* zero_point, int qmin, int qmax,
                        int index_offset, int O, int inner, uint8_t* widx, uint8_t* mask, float* q,
                        int* wsum, void* stream);

/* ---- 256-entry table maps ------------------------------------------------------------------- */
/* out[i] = table[idx(x[i])] (lut_map, approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:96-130, 793-807). */
int atb_lut_map(const void* x, int dtype, const float* table, float* out, long long numel, void* stream);
/* mapped image with constant border table[128]
 * (lut_map_pad, approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:277-311, 809-850). */
int atb_lut_map_pad(const void* x, int dtype, const float* table, float* out, int N, int C, int H, int W,
                    int ph, int pw, void* stream);

/* ---- backward: STE / LRE (256-entry slope tables) ------------------------------------------------
 * Column-space (unfolded) operands, the contract of bgemm_lre_backward_claude
 * (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:539-647):
 *   grad_x[n,k,l] = sum_o go[n,o,l] * dx[idx(w[o,k])]      grad_w[o,k] = sum_{n,l} go[n,o,l] * dw[idx(x[n,k,l])]
 * w is given as [O,K] (w_ok_layout = 1) or [K,O] (0); grad_w is written in the same layout.
 * STE is the same call with the decode table dx = dw = arange(256) - 128. */
int atb_lre_bwd(const float* go, const void* x, int x_dtype, const void* w, int w_dtype, int w_ok_layout,
                const float* dx, const float* dw, float* grad_x, float* grad_w,
                int N, int K, int L, int O, void* stream);
/* Image-space form used by the conv Functions: x is the quantised image [N,C,H,W]; grad_x is the
 * gradient w.r.t. that image (the fold is fused), grad_w is [O, C*kh*kw]; taps outside the image
 * contribute dw[pad_index] to grad_w (pad_index 0..256: 256 addresses a 257th entry the caller appended to
 * dw, for a pad value that is only known on the device).  `go_scale` (optional, [O]) multiplies go per output
 * channel.  `w_zero` (optional, [O]) is subtracted from the mapped weight, grad_x uses dx[widx[o,k]] - w_zero[o]:
 * the weight zero point of the asymmetric layer, whose correction term -z_w[o] * sum_k q_x has that derivative
 * (approxtorch/nn/Conv2d_uint8.py:308-315).
 * Runs on the tensor cores (tcgen05, fp32 operands split into three bf16 terms, fp32 accumulation in TMEM) whenever
 * every tensor is addressable with 32-bit offsets; otherwise on the fp32 SIMT kernels.
 * x_mask / x_scale (optional, together): the fake-quant backward of the activation is applied in grad_x's store,
 * grad_x = (x_mask ? g : 0) / max(*x_scale, 1e-12) (fakequant_per_tensor_backward_claude,
 * approxtorch/backend/csrc/claude/quantization.cu:113-143, without its separate 9-byte-per-element pass).
 * flags: bit 0 = dx, dw and w_zero hold integers of magnitude <= 256 (the STE decode tables): half the tensor-core
 * work; bit 1 = use the SIMT kernels; bit 2 = never pack the operands into scratch; bit 3 = with packed operands,
 * grad_w's slices of the pixel axis are stored separately and added in a fixed order by a second pass (bit-identical
 * from run to run; the default adds them with fp32 atomics in whatever order the blocks finish).
 * scratch / scratch_bytes: optional device memory of atb_lre_conv_bwd_scratch_bytes() bytes (16-byte aligned).
 * Replaces the cuDNN convolution_backward calls of approxtorch/nn/bgemm_int8.py:165-212, 259-295. */
int atb_lre_conv_bwd(const float* go, const void* x, int x_dtype, const uint8_t* widx /*[O,K]*/,
                     const float* dx, const float* dw, const float* go_scale, const float* w_zero,
                     const uint8_t* x_mask /*[N,C,H,W] or NULL*/, const float* x_scale /*scalar or NULL*/,
                     float* grad_x /*[N,C,H,W]*/, float* grad_w /*[O,K]*/,
                     int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw, int ph, int pw,
                     int dh, int dw_, int pad_index, int flags, void* scratch, size_t scratch_bytes, void* stream);
/* Bytes of device scratch with which atb_lre_conv_bwd packs its operands ahead of the contraction (the gradient is
 * split once into bf16 planes laid out the way grad_x and grad_w read them, so that the operand tiles are filled by
 * 16-byte asynchronous copies); 0 when the problem does not qualify.  With less scratch than this (or none) the same
 * call builds the operands inside the contraction kernels: same results to fp32 rounding, slower.
 * need_x / need_w: which gradients the call will ask for.  (No counterpart in the reference.) */
size_t atb_lre_conv_bwd_scratch_bytes(int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw, int ph, int pw,
                                      int dh, int dw_, int flags, int need_x, int need_w);
/* Device-side error word of the tensor-core backward (host pointer out; synchronises): 1 = a block gave up waiting
 * for its MMAs and left its tile unwritten.  (No counterpart in the reference.) */
int atb_tensor_core_status(int* status /*host*/);

/* ---- backward: custom pair tables (256x256) --------------------------------------------------------
 * grad_x[n,k,l] = sum_o dY[n,o,l] * dx_lut[x][w[o,k]]   (approxtorch/backend/csrc/cuda/bgemm_custom_grad_optimize.cu:30-116, 212-257)
 * grad_w[o,k]   = sum_{n,l} dY[n,o,l] * dw_lut[x][w]    (same file :136-205, 259-301)
 * x, w are uint8 LUT indices.  The kernels read a PREPARED copy of the table (transposed and lane-permuted for
 * their staging loads): build it once per table with atb_pair_table_prepare (atb_pair_table_bytes() bytes,
 * 16-byte aligned) and pass it as dx_prepared / dw_prepared.
 * mode: 0 = the table is held in the shared memory of a two-block cluster, half each, and read across the
 * cluster (the default); 1 = staging reads come from global memory.  Same results either way.
 * grad_w is accumulated with fp32 atomics over the pixel-row tiles (zeroed by the call). */
size_t atb_pair_table_bytes(void);
int atb_pair_table_prepare(const float* table /*[256][256], row = x*/, float* prepared, void* stream);
int atb_custom_bwd_dx(const uint8_t* x, const uint8_t* w, const float* dy, const float* dx_prepared,
                      float* grad_x, int N, int K, int L, int O, int mode, void* stream);
int atb_custom_bwd_dw(const uint8_t* x, const uint8_t* w, const float* dy, const float* dw_prepared,
                      float* grad_w, int N, int K, int L, int O, int mode, void* stream);
/* Image form of both (conv2d_int8_custom's backward, approxtorch/nn/bgemm_int8.py:105-118, without its im2col_u8
 * columns and F.fold): x is the quantised image [N,C,H,W] (int8 values or uint8 indices), taps outside it look
 * up pad_index; grad_x [N,C,H,W] is the gradient with respect to the image (fp32 atomics), grad_w is
 * [O, C*kh*kw].  Either output may be NULL. */
int atb_custom_conv_bwd(const void* x, int dtype, const uint8_t* w, const float* dy,
                        const float* dx_prepared, const float* dw_prepared, float* grad_x, float* grad_w,
                        int N, int C, int H, int W, int O, int kh, int kw, int sh, int sw, int ph, int pw,
                        int dh, int dw_, int pad_index, int mode, void* stream);
/* Device-side error word of the custom-gradient kernels (host pointer out; synchronises): 1 = a block gave up
 * waiting for its half of the table and skipped its work.  (No counterpart in the reference.) */
int atb_pair_status(int* status /*host*/);

/* ---- depthwise LUT conv (groups == C, channel multiplier 1) ----------------------------------------
 * Forward: dwconv_fake_int8_claude, approxtorch/backend/csrc/claude/dwconv_claude.cu:78-266 (taps in ascending
 * (i, j) order: bit-identical to a per-channel LUT GEMM). */
int atb_lut_dwconv_fwd(const void* x, int dtype, const uint8_t* widx /*[C, kh*kw]*/, const void* lut_image,
                       float* y, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
                       int dh, int dw, int pad_index, void* stream);
/* STE / LRE backward of the same layer on the saved 8-bit tensors:
 *   grad_x[n,c,h,w] = gs[c] * sum_taps go * dx[widx[c,t]],   grad_w[c,t] = gs[c] * sum_{n,oh,ow} go * dw[x or pad_index]
 * (dx / dw the 256-entry slope or decode tables; pad_index 256 selects a 257th entry of dw; gs optional).  Replaces
 * the lut_map + lut_map_pad + two grouped cuDNN calls of approxtorch/nn/bgemm_int8.py:189-210.  Either output may
 * be NULL; grad_w is added with fp32 atomics when a channel's pixels are split over several blocks. */
int atb_lut_dwconv_bwd(const float* go, const void* x, int dtype, const uint8_t* widx,
                       const float* dx, const float* dw_tab, const float* go_scale, float* grad_x, float* grad_w,
                       int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
                       int dh, int dw, int pad_index, void* stream);

/* ---- measurement aid (no counterpart in the reference) ---------------------------------------------
 * Launches `blocks` blocks of 1024 threads that each issue iters x 8 conflict-free 8-byte shared-memory loads
 * per thread (2 bank words each) and store a checksum to out[blocks * 1024]; timed by the caller, it gives the
 * shared-memory load rate an SM really sustains, the denominator of the LUT GEMM's roofline.
 * seed256: 256 arbitrary words. */
int atb_probe_shared_load(const unsigned* seed256, unsigned* out, int blocks, int iters, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* APPROXTORCH_B200_H */
