/*
 * geo_sc.h -- C ABI of libgeo_sc.so: the stochastic-computing (SC) conv2d / linear
 * forward hot path of nanocad-lab/geo, written for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only.  Every pointer named "device" must be device
 * memory of the current CUDA device.  The library allocates no device memory at
 * run time: the caller owns every workspace.  (Two stated exceptions: the fixed
 * LFSR tables and the 64 MiB stream scratch of geo_sc_conv2d_forward_static are
 * file-scope device arrays that come with the library image, and
 * geo_sc_measure_lop3_peak allocates and frees a few bytes.)  It never throws and
 * never traps: every entry point returns GEO_SC_OK (0) or a negative
 * geo_sc_status, and geo_sc_last_error() gives a thread-local human-readable
 * detail.  Entry points may be called from several host threads at once; work
 * given to different streams is independent unless an entry point says otherwise.  All work is enqueued on the
 * stream passed in (a cudaStream_t passed as void*; NULL = default stream) and
 * the call returns without synchronising.  The one exception is the first call
 * on each device, which uploads the LFSR pattern tables with a synchronous copy;
 * make that first call (or geo_sc_init) before any stream capture.
 *
 * Each entry point cites the reference interface it replaces
 * (paths relative to the reference project root).
 */
#ifndef GEO_SC_H
#define GEO_SC_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GEO_SC_VERSION 1

/* Accumulation modes (which filter axes are OR-accumulated inside a group and
 * which are added in binary across groups). */
#define GEO_SC_MODE_1D 0      /* OR over (c,ky), add over kx: sc_cuda_kernel.cu:590-1004, sc.cpp:292-472 */
#define GEO_SC_MODE_Z 1       /* OR over (ky,kx), add over c: sc_cuda_kernel.cu:1141-1271                */
#define GEO_SC_MODE_YZ 2      /* OR over (c mod z,ky), add over (c div z,kx): sc_cuda_kernel.cu:1007-1138 */
#define GEO_SC_MODE_FULL_OR 3 /* OR over (c,ky,kx): utils_functional.py:554-609 (LFSR, deterministic)     */
#define GEO_SC_MODE_2D 4      /* OR over c, add over (ky,kx): utils_functional.py:528-541,597-601 (only in
                                 the reference's bit-serial simulation; weight generators indexed by c)  */
#define GEO_SC_MODE_FULL_BIN 5 /* no OR at all: every product bit is counted (utils_functional.py:593-595,607-609,
                                 simulation only); the guide is the plain convolution (:617-619)        */

/* Stream generators.  LFSR: the reference's deterministic generator (sc_cuda_kernel.cu:18-40,156-167), the
 * only one with bit-exact parity.  ACC: the "accurate" generator of the reference (utils_functional.py:63-73,
 * 157-176; cuRAND in sc_cuda_kernel.cu:354-417): sampling without replacement, so that a stream of level V
 * holds exactly V ones; every activation element and every weight has its own generator (nothing is shared),
 * progressive loading does not apply.  Here it is counter-based (a hash of seed, element and bit index), hence
 * reproducible; against the reference, whose generators are random, parity is statistical only. */
#define GEO_SC_GEN_LFSR 0
#define GEO_SC_GEN_ACC 1
/* RAND: the "true random" generator of the reference's simulation (utils_functional.py:92-102,148-150): every
 * bit compares the level with a fresh uniform integer below bit_length, so the bits of a stream are independent
 * with probability level / bit_length; the integers are shared the way the LFSR generators are (weights over
 * c_out and the binary-accumulated axis, activations over the batch).  Counter-based like ACC, statistical
 * parity only. */
#define GEO_SC_GEN_RAND 2

typedef enum geo_sc_status {
    GEO_SC_OK = 0,
    GEO_SC_ERR_NULL = -1,        /* a required pointer is NULL                                  */
    GEO_SC_ERR_BIT_LENGTH = -2,  /* bit_length not in {8,16,32,64,128,256}                      */
    GEO_SC_ERR_SHAPE = -3,       /* a dimension is < 1, or the filter is larger than the image  */
    GEO_SC_ERR_MODE = -4,        /* unknown accumulation mode                                   */
    GEO_SC_ERR_LOADING = -5,     /* total_width / load_width / load_wait out of range           */
    GEO_SC_ERR_TOO_LARGE = -6,   /* an index would not fit 31 bits                              */
    GEO_SC_ERR_WORKSPACE = -7,   /* workspace smaller than geo_sc_*_bytes reports, or unaligned */
    GEO_SC_ERR_CUDA = -8,        /* a CUDA runtime call failed (detail in geo_sc_last_error)    */
    GEO_SC_ERR_UNSUPPORTED = -9  /* valid request that this build does not implement            */
} geo_sc_status;

/*
 * One SC convolution.  Activations are fp32 NCHW [batch][c_in][h_in][w_in], weights
 * fp32 [c_out][c_in][k_h][k_w], output int32 [batch][c_out][h_in+2*pad_h-k_h+1][w_in+2*pad_w-k_w+1]
 * holding (positive count - negative count) over all stream bits.  Stride is 1
 * (the reference accepts a stride argument and ignores it, sc_cuda_kernel.cu:1732-1834).
 * Zero padding is applied to dim 2 by pad_h and dim 3 by pad_w before anything else
 * (what F::pad does in sc_cuda.cpp:50); generator seeds are indexed in padded coordinates.
 *
 * total_width / load_width / load_wait_*: progressive loading
 * (sc_cuda_kernel.cu:156-160,682-685): for 1-based stream bit t the visible width is
 * min(total_width, (t / load_wait + 1) * load_width - 1).  load_width >= total_width + 1
 * disables it.  load_wait_w applies to weight streams, load_wait_a to activation
 * streams (they differ only in yz mode, sc_cuda_kernel.cu:2021,2104).
 * z_unit is used by GEO_SC_MODE_YZ only and is clamped to c_in
 * (sc_cuda_kernel.cu:1987).
 */
typedef struct geo_sc_conv_desc {
    int32_t batch, c_in, h_in, w_in;
    int32_t pad_h, pad_w;
    int32_t c_out, k_h, k_w;
    int32_t bit_length;
    int32_t mode;
    int32_t z_unit;
    int32_t total_width, load_width, load_wait_w, load_wait_a;
    int32_t generator;   /* GEO_SC_GEN_LFSR (0, the default of a zero-initialised tail), _ACC or _RAND */
    uint32_t seed;       /* _ACC and _RAND: selects the random streams; the same seed repeats them */
} geo_sc_conv_desc;

int geo_sc_version(void);
const char *geo_sc_status_string(int status);
/* Detail of the last failure on the calling thread ("" if none). */
const char *geo_sc_last_error(void);

/* Uploads the LFSR pattern tables to the current device (idempotent).  Called
 * implicitly by the first generation call on a device. */
int geo_sc_init(void);

/* Kernels of this library that wait on hardware barriers (the tcgen05 / TMA kernels of the guide) bound every wait;
 * a wait that runs out makes its thread block give up and raises a device-side count.  *count receives that count
 * for the current device since the library was loaded: 0 in a healthy run, anything else means that the results
 * of some guide call are not to be trusted.  Synchronises with the device (a small device-to-host copy).  No
 * counterpart in the reference. */
int geo_sc_device_error_count(int *count);

/* ---- whole forward --------------------------------------------------------------
 * Replaces sc_extension_cuda.conv2d_add_partial_variable_acc (sc_cuda.cpp:47-63; dim==0 ->
 * GEO_SC_MODE_Z, else GEO_SC_MODE_1D), conv2d_add_yz_variable_acc (sc_cuda.cpp:34-45) and,
 * with the deterministic LFSR generator, conv2d_or_acc (sc_cuda.cpp:21-32); on CPU tensors
 * the reference calls sc_extension.conv2d_add_partial_new (sc.cpp:292-472) for the same
 * 1d mode.  Quantisation (sc_cuda.cpp:51-55), padding, stream generation and the
 * AND/OR/popcount accumulation all happen inside.  workspace: device, 256-byte aligned,
 * at least geo_sc_conv2d_workspace_bytes. */
int geo_sc_conv2d_workspace_bytes(const geo_sc_conv_desc *desc, size_t *bytes);
int geo_sc_conv2d_forward(const geo_sc_conv_desc *desc, const float *act_device, const float *weight_device,
                          int32_t *out_device, void *workspace_device, size_t workspace_bytes, void *stream);

/* ---- whole forward without a workspace argument -----------------------------------------
 * No counterpart in the reference (whose launchers allocate managed memory on every call).
 * For hosts that cannot give the library device memory at call time -- a runtime whose memory
 * plan is frozen, a loop that must not touch the allocator once it is running, a plugin
 * interface that carries tensor pointers only -- the stream scratch of this variant is a fixed
 * array of geo_sc_static_scratch_bytes() = 64 MiB inside the library, resident on every GPU
 * that loads it until the process exits.  It performs no device allocation of any kind; the
 * caller still passes act, weight and out.  Same results as geo_sc_conv2d_forward.
 *   - A convolution whose streams need more than the array is refused with
 *     GEO_SC_ERR_WORKSPACE (the message gives both sizes).
 *   - All calls share the array and it keeps whatever the previous call left; each call
 *     rewrites every word it later reads, so that is harmless for calls that run one after
 *     another, but two calls that may overlap on the GPU (other streams, other threads) race.
 *   - The first call on each device looks up the array's device address (and, like every entry
 *     point, may upload the LFSR tables): make it before starting any stream capture.
 *   - It always runs the dense accumulation kernel, because the sign-sorted weight section would
 *     take scratch of its own: layers with long groups (64 or more members per group) give the
 *     same result through it but run about a quarter slower than through geo_sc_conv2d_forward. */
size_t geo_sc_static_scratch_bytes(void);
int geo_sc_conv2d_forward_static(const geo_sc_conv_desc *desc, const float *act_device, const float *weight_device,
                                 int32_t *out_device, void *stream);

/* Which accumulation kernel serves this descriptor: *yes = 1 for a sign-sorted kernel (the members of a
 * group, or of a 16-member chunk of it where groups are short, are sorted per four output channels by the
 * signs of their weights when the weights are prepared, and each weight costs one 32-bit logic op per
 * activation word instead of the two of the dense form), 0 for the dense kernel.  Results are identical;
 * the figure matters only for counting executed logic ops. */
int geo_sc_accumulate_is_sign_sorted(const geo_sc_conv_desc *desc, int *yes);

/* The same choice by name: *kernel = one of the values below.  No counterpart in the reference (it has one
 * kernel); used by the benchmarks to label their rows and by the tests to know which kernel a case exercises. */
#define GEO_SC_KERNEL_DENSE 0          /* sc_accumulate.cu */
#define GEO_SC_KERNEL_SORTED_IM2COL 1  /* sc_accumulate_sorted.cu */
#define GEO_SC_KERNEL_SORTED_ROWS 2    /* sc_accumulate_rows.cu */
#define GEO_SC_KERNEL_SORTED_SHORT 3   /* sc_accumulate_short.cu */
#define GEO_SC_KERNEL_FULL_BIN 4       /* sc_accumulate_fullbin.cu */
#define GEO_SC_KERNEL_SORTED_TAPS 5    /* sc_accumulate_taps.cu */
int geo_sc_accumulate_kernel(const geo_sc_conv_desc *desc, int *kernel);

/* ---- the three stages, for callers that cache weight streams across calls ---------
 * (weights change once per optimiser step and never during evaluation).
 *
 * geo_sc_prepare_weights replaces the stream_generation_transpose_* kernels
 * (sc_cuda_kernel.cu:91-349).  Prepared layout: uint32 words
 * [pack][group][member_padded][c_out_padded][2] (last index 0 = positive stream, seed base 67;
 * 1 = negative, base 37), followed by an int32 table [group][member_padded] of activation
 * offsets; members are padded (see geo_sc_group_geometry) with zero streams, c_out_padded = c_out
 * rounded up to the kernel's c_out tile
 * (see geo_sc_group_geometry).  Bits are MSB-first inside a word, 32 per pack.  A third section follows for
 * the sign-sorted accumulate kernel that the layer's geometry selects (geo_sc_accumulate_kernel): per
 * (group, chunk of members, quad of four output channels) the members sorted by which of the four
 * weights are negative -- one uint4 with the four non-zero stream words per member and pack, the member's
 * offset in the kernel's tile and the boundaries of the 16 patterns; the chunking (whole groups of planes,
 * filter taps x channels, or 16 members) and the widths of the offsets differ per kernel and are
 * private to the library; geo_sc_weight_prep_bytes covers all three sections.
 * For GEO_SC_MODE_FULL_BIN the third section holds the weight words once more, in the order the binary
 * tensor-core GEMM of that mode reads them (tiles of 32 output channels x 2 polarities x 32 words).
 * Neither the size nor the contents of the prepared buffer depend on `batch`: a buffer prepared once
 * serves geo_sc_accumulate calls of any batch size whose descriptor agrees in every other field
 * (geo_sc_accumulate picks the dense or the sign-sorted kernel per call; both sections are there).
 *
 * geo_sc_generate_act_streams replaces the generation loops at
 * sc_cuda_kernel.cu:667-691,1079-1102,1218-1236 and the quantise/pad ops in sc_cuda.cpp.
 * Layout: uint32 words [batch][pack][c_in][h_in+2*pad_h][w_in+2*pad_w], or -- for the descriptors for which
 * geo_sc_act_stream_layout says so -- batch-innermost [pack][c_in][h_in+2*pad_h][w_in+2*pad_w][batch_padded]
 * with the batch rounded up to a multiple of 4 and the images past it all zero: the same pixel of
 * consecutive images is then consecutive words (linear layers, whose positions are the images).  A stream
 * buffer is only valid for the descriptor (batch included) it was generated with.
 *
 * geo_sc_accumulate replaces stream_compute_add_direct_variable (:694-1002) and
 * matmul_outer (:43-86); it picks the dense or the sign-sorted kernel from the descriptor alone. */
int geo_sc_weight_prep_bytes(const geo_sc_conv_desc *desc, size_t *bytes);
int geo_sc_prepare_weights(const geo_sc_conv_desc *desc, const float *weight_device, void *wprep_device,
                           size_t wprep_bytes, void *stream);
int geo_sc_act_stream_bytes(const geo_sc_conv_desc *desc, size_t *bytes);
int geo_sc_act_stream_layout(const geo_sc_conv_desc *desc, int *batch_innermost, int *batch_padded);
int geo_sc_generate_act_streams(const geo_sc_conv_desc *desc, const float *act_device, void *astream_device,
                                size_t astream_bytes, void *stream);
int geo_sc_accumulate(const geo_sc_conv_desc *desc, const void *astream_device, const void *wprep_device,
                      int32_t *out_device, void *stream);

/* Geometry of the prepared-weight layout: groups, members per group (logical, and as laid out:
 * rounded up to a multiple of 4 (up to 16 members) or of 16, with all-zero streams), c_out tile,
 * padded c_out. */
int geo_sc_group_geometry(const geo_sc_conv_desc *desc, int32_t *groups, int32_t *members, int32_t *members_padded,
                          int32_t *cout_tile, int32_t *cout_padded);

/* ---- SC linear layer ---------------------------------------------------------------
 * act [batch][features] . weight [out_features][features]^T with OR accumulation inside
 * groups of z_unit consecutive inputs and binary accumulation across groups.  The
 * reference has no native kernel for it (utils_functional.py:302-404 is a bit-serial
 * PyTorch loop); it is defined here as GEO_SC_MODE_YZ on a 1x1 image, which is what it
 * reduces to.  desc: batch, c_in = features, c_out = out_features, bit_length, z_unit and
 * the loading fields are read; h_in, w_in, k_h, k_w must be 1 and pads 0. */
int geo_sc_linear_forward(const geo_sc_conv_desc *desc, const float *act_device, const float *weight_device,
                          int32_t *out_device, void *workspace_device, size_t workspace_bytes, void *stream);

/* ---- float guide: the straight-through backward used for training ------------------------
 * Replaces what the reference gets from PyTorch autograd over its guide functions
 * (utils_functional.py:189-296 and :611-634): with w+ = clamp(w,0,100), w- = -clamp(w,-100,0)
 * and y(+/-)_g the plain fp32 convolution restricted to binary-accumulated group g,
 *     out = sum_g (1 - exp(-y+_g)) - sum_g (1 - exp(-y-_g)),
 * whose value the caller replaces by the SC result and whose gradient is the layer's gradient.
 *
 * The guide's value is never needed, only its gradient, so there is a single entry point for the
 * backward pass: from act [batch][c_in][h_in][w_in], weight and grad_out [batch][c_out][Ho][Wo]
 * it produces grad_act (same shape as act) and/or grad_weight [c_out][c_in][k_h][k_w]; either may
 * be NULL = not wanted.  scratch: device, 256-byte aligned, geo_sc_guide_backward_bytes.
 * All fp32, no atomics: results are run-to-run deterministic. */
int geo_sc_guide_backward_bytes(const geo_sc_conv_desc *desc, size_t *scratch_bytes);
int geo_sc_guide_backward(const geo_sc_conv_desc *desc, const float *act_device, const float *weight_device,
                          const float *grad_out_device, float *grad_act_device, float *grad_weight_device,
                          void *scratch_device, size_t scratch_bytes, void *stream);
/* Same call for a caller that has already quantised act and weight the way the reference's layer
 * does before it calls the guide (Conv2d_Add_Partial.forward, utils_class.py:190-204: multiples of
 * 2^-prec with prec <= 8 inside [-1, 1], which bf16 holds exactly).  For the 1d_bin and full_or
 * modes only the tensor-core kernels are then launched; should the promise not hold (checked on
 * the device) the requested gradients are filled with NaN instead of being computed by the fp32
 * kernels.  Other modes behave exactly like geo_sc_guide_backward. */
int geo_sc_guide_backward_quantized(const geo_sc_conv_desc *desc, const float *act_device, const float *weight_device,
                                    const float *grad_out_device, float *grad_act_device, float *grad_weight_device,
                                    void *scratch_device, size_t scratch_bytes, void *stream);

/* ---- quantised batch normalisation between SC layers -------------------------------------------
 * Replaces BatchNorm2d_fixed / BatchNorm1d_fixed (utils_class.py:37-93), which the reference
 * evaluates as F.batch_norm plus separate mean/var reductions and a chain of small element-wise
 * ops (quantize_shift, utils_functional.py:41-57).  x and out are [batch][channels][spatial]
 * (spatial = H*W, or 1 for the 1d layer).  Forward value: x * w_q + b_q with the folded scale
 * w_n = weight / sqrt(var + eps) and shift b_n = bias - mean * weight / sqrt(var + eps) rounded to
 * 7 bits under the common range scale = 2^ceil(log2(3 * mean_c(w_n))) (written to scale_out[0]);
 * in training mode mean/var are the biased batch statistics and running_mean / running_var are
 * updated with `momentum` (unbiased variance), in evaluation mode the running statistics are used.
 * save_mean / save_invstd [channels] feed the backward pass, which is the gradient of the
 * unquantised normalisation (what the reference's graph differentiates).  weight / bias may be
 * NULL (no affine); grad_weight / grad_bias may be NULL.  Reductions are two-level and
 * order-fixed: results are run-to-run deterministic. */
int geo_sc_bn_fixed_scratch_bytes(int batch, int channels, size_t *bytes);
int geo_sc_bn_fixed_forward(int batch, int channels, int spatial, int training, float eps, float momentum,
                            const float *x_device, const float *weight_device, const float *bias_device,
                            float *running_mean_device, float *running_var_device, float *out_device,
                            float *save_mean_device, float *save_invstd_device, float *scale_out_device,
                            void *scratch_device, size_t scratch_bytes, void *stream);
int geo_sc_bn_fixed_backward(int batch, int channels, int spatial, int training, const float *x_device,
                             const float *grad_out_device, const float *weight_device, const float *save_mean_device,
                             const float *save_invstd_device, float *grad_x_device, float *grad_weight_device,
                             float *grad_bias_device, void *scratch_device, size_t scratch_bytes, void *stream);

/* ---- batch norm + 2x2 average pool + hardtanh(0, 1) as one pass per direction ---------------------
 * Replaces the sequence bn -> nn.AvgPool2d(2) -> nn.Hardtanh(0, 1) between the reference's SC layers
 * (network.py:168-184 over utils_class.py:37-65).  x [batch][channels][height][width], out and
 * grad_out [batch][channels][height/2][width/2]; even height, width a multiple of 4, x / grad_x
 * 16-byte and the pooled tensors 8-byte aligned (GEO_SC_ERR_SHAPE otherwise: use the separate entry
 * points).  Value and gradients equal the composition of geo_sc_bn_fixed_* and geo_sc_pool_act_*;
 * the normalised tensor and its gradient are never stored.  save_wq / save_bq [channels] receive the
 * folded, quantised scale and shift that the backward pass needs to recompute the pooled value.
 * scratch as for geo_sc_bn_fixed_forward. */
int geo_sc_bn_pool_act_forward(int batch, int channels, int height, int width, int training, float eps, float momentum,
                               const float *x_device, const float *weight_device, const float *bias_device,
                               float *running_mean_device, float *running_var_device, float *out_device,
                               float *save_mean_device, float *save_invstd_device, float *save_wq_device,
                               float *save_bq_device, float *scale_out_device, void *scratch_device,
                               size_t scratch_bytes, void *stream);
int geo_sc_bn_pool_act_backward(int batch, int channels, int height, int width, int training, const float *x_device,
                                const float *grad_out_device, const float *weight_device,
                                const float *save_mean_device, const float *save_invstd_device,
                                const float *save_wq_device, const float *save_bq_device, float *grad_x_device,
                                float *grad_weight_device, float *grad_bias_device, void *scratch_device,
                                size_t scratch_bytes, void *stream);

/* ---- from the bit counts of one SC layer to the packed streams of the next, one pass ---------------------
 * Replaces the whole chain the reference runs between two SC layers (network.py:165-184): result / bit_length
 * (utils_functional.py:632-634) -> BatchNorm2d_fixed (utils_class.py:37-65) -> nn.AvgPool2d(2) -> nn.Hardtanh(0, 1)
 * -> quantize of the next layer's input (utils_class.py:32, utils_functional.py:33-39) -> float -> level and stream
 * generation of the next layer (sc_cuda.cpp:50-51, sc_cuda_kernel.cu:667-691).  next_desc describes the NEXT layer:
 * its batch, c_in, h_in, w_in are the pooled tensor, counts is int32 [batch][c_in][2*h_in][2*w_in] (w_in even,
 * counts 16-byte aligned); in_bit_length is the stream length the counts were produced with; prec the fractional
 * bits of the rounding (the reference uses 7).  The batch-norm statistics are taken over counts / in_bit_length
 * exactly as geo_sc_bn_pool_act_forward takes them over x, so every output equals what the separate entry points
 * (geo_sc_counts_to_float, geo_sc_bn_pool_act_forward, geo_sc_quantize, geo_sc_generate_act_streams) give, bit
 * for bit: act_out [batch][c_in][h_in][w_in] is the rounded activation (the next layer's backward pass reads
 * it), astream the next layer's activation streams (geo_sc_act_stream_bytes(next_desc)), save_* / scale_out /
 * scratch as for geo_sc_bn_pool_act_forward.  LFSR generator only.
 * The backward pass of the chain is geo_sc_epilogue_backward: geo_sc_bn_pool_act_backward reading the counts
 * in place of x (counts [batch][channels][height][width], the layer's own output size). */
int geo_sc_epilogue_forward(const geo_sc_conv_desc *next_desc, int in_bit_length, int prec, int training, float eps,
                            float momentum, const int32_t *counts_device, const float *weight_device,
                            const float *bias_device, float *running_mean_device, float *running_var_device,
                            float *act_out_device, float *save_mean_device, float *save_invstd_device,
                            float *save_wq_device, float *save_bq_device, float *scale_out_device, void *astream_device,
                            size_t astream_bytes, void *scratch_device, size_t scratch_bytes, void *stream);
int geo_sc_epilogue_backward(int batch, int channels, int height, int width, int in_bit_length, int training,
                             const int32_t *counts_device, const float *grad_out_device, const float *weight_device,
                             const float *save_mean_device, const float *save_invstd_device, const float *save_wq_device,
                             const float *save_bq_device, float *grad_x_device, float *grad_weight_device,
                             float *grad_bias_device, void *scratch_device, size_t scratch_bytes, void *stream);

/* ---- fixed-point rounding of activations and weights ----------------------------------------------
 * Replaces quantize (utils_functional.py:33-39), which the reference evaluates as four element-wise
 * PyTorch ops: y = clamp(round_half_even(x * 2^prec), -(2^prec - 1), 2^prec - 1) / 2^prec, one kernel.
 * x and y: device, n floats; y may be x.  prec 0..23. */
int geo_sc_quantize(const float *x_device, float *y_device, size_t n, int prec, void *stream);

/* The hand-off from bit counts to the layer's value (utils_functional.py:497-498, 632-634:
 * result.float() / bit_length written over the guide's output), one kernel: out = counts / bit_length,
 * exact because bit_length is a power of two.  counts and out: device, n elements. */
int geo_sc_counts_to_float(const int32_t *counts_device, float *out_device, size_t n, int bit_length, void *stream);

/* 2x2 average pooling (stride 2, a trailing odd row or column is dropped) followed by
 * hardtanh(0, 1): the activation the reference puts between SC layers (network.py:168-184,
 * nn.AvgPool2d(2) then nn.Hardtanh(0,1)), one pass per direction.  x is [planes][height][width]
 * (planes = batch * channels), y [planes][height/2][width/2].  The backward pass recomputes the
 * pooled value from x; the gradient passes where it lies strictly inside (0, 1). */
int geo_sc_pool_act_forward(int planes, int height, int width, const float *x_device, float *y_device, void *stream);
int geo_sc_pool_act_backward(int planes, int height, int width, const float *x_device, const float *grad_y_device,
                             float *grad_x_device, void *stream);

/* ---- host mirror of the stream generator ------------------------------------------------
 * Runs on the CPU with the same pattern tables and loading plan the kernels use, for one
 * integer level `value` in [0, bit_length): seed = (seed_base + seed_index) mod (L-1) + 1
 * (sc_cuda_kernel.cu:1757-1763,668-670), bits as in sc_cuda_kernel.cu:151-168.  Writes
 * ceil(bit_length/32) words.  Needs no GPU. */
int geo_sc_host_stream(int bit_length, int value, int seed_base, int seed_index, int total_width, int load_width,
                       int load_wait, uint32_t *words);

/* ---- measurement helper ---------------------------------------------------------------
 * Runs an unrolled chain of independent 32-bit LOP3 instructions on every SM and
 * reports the measured rate in 32-bit logic ops per second (the integer-pipe roofline
 * denominator).  Synchronises the device and, unlike every other entry point, allocates
 * (and frees) a few bytes of device memory.  No counterpart in the reference. */
int geo_sc_measure_lop3_peak(double *lop3_per_second, double *milliseconds);

#ifdef __cplusplus
}
#endif
#endif /* GEO_SC_H */
