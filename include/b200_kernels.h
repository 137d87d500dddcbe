/*
 * b200_kernels.h - C ABI of the B200 (sm_100a) quantized-inference kernels.
 *
 * This is the boundary between host code (the nGraph backend plugin, or any
 * other caller) and the hand-written CUDA kernels.  Plain pointers and sizes
 * only: no C++ types, no exceptions, no framework types.  Unless a function
 * says otherwise every data pointer is a DEVICE pointer valid on the current
 * CUDA device and `stream` is a cudaStream_t passed as void* (NULL = the
 * legacy default stream).  Calls are asynchronous with respect to the host.
 *
 * Every entry point returns a b200_status: 0 on success, a negative value
 * for an argument the kernel cannot run (nothing is launched), a positive
 * value for a CUDA runtime/driver error.  There is no CPU fallback: when
 * there is no usable GPU the functions return B200_ERR_CUDA.
 *
 * Each declaration cites the interface of the nGraph reference
 * (path:line inside the ngraph source tree) whose arithmetic it reproduces.
 */
#ifndef B200_KERNELS_H
#define B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

typedef enum b200_status
{
    B200_OK = 0,
    B200_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad rank, bad enum            */
    B200_ERR_UNSUPPORTED = -2,      /* legal in nGraph, not implemented on device  */
    B200_ERR_TOO_LARGE = -3,        /* exceeds a documented size limit             */
    B200_ERR_DEVICE_STATUS = -4,    /* a kernel gave up on a bounded wait          */
    B200_ERR_CUDA = 1               /* cudaGetLastError() / driver error           */
} b200_status;

/* Element types, a subset of ngraph::element::Type_t (src/ngraph/type/element_type.hpp:40-59). */
typedef enum b200_dtype
{
    B200_U8 = 0,
    B200_I8 = 1,
    B200_I32 = 2,
    B200_F32 = 3,
    B200_I64 = 4 /* index tensors only (b200_gather_rows_b32) */
} b200_dtype;

/* OR-ed into the data / activation type argument of b200_qgemm* and b200_qconv*: the weights (filters) are u8, not i8
 * (op::v0::QuantizedDot / QuantizedConvolution accept u8 x u8; the fused ops do not). */
#define B200_WEIGHTS_U8 0x100


/* Same ordinal order as op::v0::Quantize::RoundMode (src/ngraph/op/quantize.hpp:38-81). */
typedef enum b200_round_mode
{
    B200_ROUND_NEAREST_TOWARD_INFINITY = 0,
    B200_ROUND_NEAREST_TOWARD_ZERO = 1,
    B200_ROUND_NEAREST_UPWARD = 2,
    B200_ROUND_NEAREST_DOWNWARD = 3,
    B200_ROUND_NEAREST_TOWARD_EVEN = 4,
    B200_ROUND_TOWARD_INFINITY = 5,
    B200_ROUND_TOWARD_ZERO = 6,
    B200_ROUND_UP = 7,
    B200_ROUND_DOWN = 8
} b200_round_mode;

#define B200_MAX_RANK 8

/* Human readable text for a status code (static storage). */
B200_API const char* b200_status_string(int status);

/* Text of the last CUDA error seen by this library on the calling thread (static storage). */
B200_API const char* b200_last_cuda_error(void);

/* Number of kernels this library has launched since load (or since the last reset). */
B200_API uint64_t b200_launch_count(void);
B200_API void b200_reset_launch_count(void);

/*
 * Reads and clears the device status word the contraction kernels set when one of their
 * bounded waits (mbarrier / TMEM) gives up instead of hanging.  Synchronises with the device.
 * Returns B200_OK (and *status_out = 0) or B200_ERR_DEVICE_STATUS (and the code in *status_out).
 */
B200_API int b200_device_status(int* status_out);

/*
 * Self-test of that give-up path (diagnostic; no reference counterpart - nGraph's backends have no device-side waits).
 * Queues one small kernel whose single waiting thread polls, through the same bounded wait the contraction kernels
 * use, an mbarrier that nothing arrives at.  After limit_ns (1 .. 100 000 000) the wait gives up, the kernel stores
 * code 9001 in the device status word and returns normally; the context stays usable.  The next b200_device_status()
 * then returns B200_ERR_DEVICE_STATUS once (and the plugin's Tensor::read throws once).  Nothing traps or spins forever.
 */
B200_API int b200_selftest_bounded_wait(int64_t limit_ns, void* stream);

/*
 * Quantize: f32 -> u8 / i8 / i32.
 *
 * Replaces runtime::reference::quantize<float,QUANT>
 * (src/ngraph/runtime/reference/quantize.hpp:30-117) as dispatched by the
 * INTERPRETER for op::v0::Quantize (src/ngraph/runtime/interpreter/int_executable.hpp:1405-1451).
 *
 *   q = x / scale[proj]            IEEE single-precision division
 *   q = round(q)                   per round_mode, the literal floor/ceil(+-0.5) sequences
 *   q = q + (float)zero_point[proj]
 *   q = clamp(q, QUANT::min, QUANT::max);  out = (QUANT)q
 *
 * `shape`/`rank` describe the row-major input; `axes` (ascending, n_axes of
 * them) are the quantisation axes, scale and zero_point are row-major tensors
 * over exactly those axes (n_axes == 0: one element each).  zero_point has
 * the output element type.  A NaN input produces 0.
 */
B200_API int b200_quantize(const float* input,
                           const float* scale,
                           const void* zero_point,
                           void* output,
                           int quant_type, /* b200_dtype: U8, I8 or I32 */
                           const int64_t* shape,
                           int rank,
                           const int64_t* axes,
                           int n_axes,
                           int round_mode, /* b200_round_mode */
                           void* stream);

/*
 * Quantize to 8 bits with ROUND_NEAREST_TOWARD_EVEN normally replaces the per-element IEEE division
 * by a per-row correctly rounded reciprocal plus two fused multiply-adds that reproduce the correctly
 * rounded quotient bit for bit (see quantize.cu).  b200_set_fast_division(0) makes every Quantize use
 * the plain division instead (the tests compare the two over all 2^32 inputs); returns the old setting.
 */
B200_API int b200_set_fast_division(int enable);

/*
 * Dequantize: u8 / i8 / i32 -> f32.
 *
 * Replaces runtime::reference::dequantize<QUANT,float>
 * (src/ngraph/runtime/reference/dequantize.hpp:32-52), INTERPRETER case at
 * src/ngraph/runtime/interpreter/int_executable.hpp:830-862.
 *
 *   out = (float)(in - zero_point[proj]) * scale[proj]
 */
B200_API int b200_dequantize(const void* input,
                             const float* scale,
                             const void* zero_point,
                             float* output,
                             int quant_type, /* b200_dtype: U8, I8 or I32 */
                             const int64_t* shape,
                             int rank,
                             const int64_t* axes,
                             int n_axes,
                             void* stream);

/*
 * Epilogue shared by the int8 contractions.  For accumulator acc (int32):
 *
 *   fused (round_half_away == 0), the contract of the experimental fused ops as the
 *   CPU backend hands it to oneDNN (src/ngraph/runtime/cpu/builder/quantized_conv.cpp:455-474,
 *   src/ngraph/runtime/cpu/dnnl_emitter.hpp:679-695,737-761), results pinned by
 *   test/builder_quantization.cpp:146-492,995-1098:
 *       v = (float)(acc + bias[n]) * scale[n or 0]
 *       v = v + sum_scale * (float)sum_in            (only when sum_in != NULL)
 *       v = max(v, 0)                                (only when relu)
 *       out = f32: v        u8/i8: saturate(round_half_even(v))      i32: (int32) the same
 *
 *   core (round_half_away == 1), the requantisation of runtime::reference::dot /
 *   convolution (src/ngraph/runtime/reference/dot.hpp:152-159,
 *   src/ngraph/runtime/reference/convolution.hpp:252-258):
 *       out = saturate( (OUT)roundf((float)acc * scale[0]) + out_zero_point )
 *   (the reference does not saturate: an out-of-range cast there is undefined behaviour).
 *
 *   raw (round_half_away == 2): out = acc, int32, exact (out_type must be I32; scale, bias, sum_in and relu are not
 *   used).  The first stage of contractions with non-zero zero points, see b200_requant_zero_points.
 *
 * All float steps are separate IEEE operations (no fused multiply-add).
 */
typedef struct b200_epilogue
{
    const int32_t* bias;   /* [N] or NULL                                             */
    const float* scale;    /* [scale_count], device memory (never an immediate)       */
    int64_t scale_count;   /* 1 (per tensor) or N (per output channel)                */
    const void* sum_in;    /* same shape/layout as the output, or NULL                */
    int sum_type;          /* b200_dtype of sum_in: U8 or I8                          */
    const float* sum_scale;/* one element, device memory; required with sum_in        */
    int relu;              /* 0 / 1                                                   */
    int round_half_away;   /* 0 = fused-op contract (RNE), 1 = core-op contract, 2 = raw */
    int32_t out_zero_point;/* core contract only                                      */
    int out_type;          /* b200_dtype: U8, I8, I32 or F32                          */
} b200_epilogue;

/*
 * Int8 matrix product with fused epilogue on the tcgen05 tensor cores.
 *
 *   acc[m,n] = sum_k A[m,k] * W[n,k]       A: [M,K] u8 or i8, W: [N,K] i8, both row-major
 *   out[m,n] = epilogue(acc[m,n])          out: [M,N] row-major
 *
 * Replaces op::v0::QuantizedDotBias as the CPU backend runs it
 * (src/ngraph/op/experimental/quantized_dot_bias.cpp:27-56,
 * src/ngraph/runtime/cpu/builder/quantized_dot.cpp:36-125) and, with the core
 * epilogue and W = transpose(B), op::v0::QuantizedDot with zero zero-points
 * (src/ngraph/op/quantized_dot.cpp:58-201, src/ngraph/runtime/reference/dot.hpp:38-167).
 *
 * K must be a multiple of 16 and all of A, W 16-byte aligned.
 */
B200_API int b200_qgemm(const void* A,
                        int a_type, /* B200_U8 or B200_I8 */
                        const int8_t* W,
                        void* out,
                        int64_t M,
                        int64_t N,
                        int64_t K,
                        const b200_epilogue* epilogue,
                        void* stream);

/*
 * Int8 2-D convolution (implicit GEMM on tcgen05) with fused epilogue.
 *
 *   data    [N,H,W,C]    u8 (or i8), channels-last, C a multiple of 16
 *   filters [K,R,S,C]    i8, channels-last
 *   out     [N,P,Q,K]    channels-last; P,Q from the usual convolution arithmetic
 *   sum_in  [N,P,Q,K]    (epilogue.sum_in) when used
 *
 * Replaces op::v0::QuantizedConvolutionBias / ...BiasAdd / ...BiasSignedAdd /
 * QuantizedConvolutionRelu (src/ngraph/op/experimental/quantized_conv_bias.cpp:26-237,
 * src/ngraph/op/experimental/quantized_conv_relu.cpp:25-80) as the CPU backend runs
 * them (src/ngraph/runtime/cpu/builder/quantized_conv.cpp:414-754), and the
 * accumulation of runtime::reference::general_convolution with zero zero-points
 * (src/ngraph/runtime/reference/convolution.hpp:59-265): padding positions contribute 0.
 * The nGraph ops are NCHW/KCRS; b200_nchw_to_nhwc_u8 / b200_nhwc_to_nchw_u8 convert.
 */
typedef struct b200_conv_params
{
    int64_t N, H, W, C; /* data                                        */
    int64_t K, R, S;    /* filters                                     */
    int64_t stride_h, stride_w;
    int64_t pad_h, pad_w;           /* padding below                    */
    int64_t pad_h_above, pad_w_above;
    int64_t dilation_h, dilation_w; /* window dilation                  */
} b200_conv_params;

B200_API int b200_qconv(const void* data,
                        int data_type, /* B200_U8 or B200_I8 */
                        const int8_t* filters,
                        void* out,
                        const b200_conv_params* params,
                        const b200_epilogue* epilogue,
                        void* stream);

/* Output spatial size of b200_qconv for the given params. */
B200_API int b200_qconv_out_shape(const b200_conv_params* params, int64_t* P, int64_t* Q);

/*
 * Layout conversions for 1-byte tensors between nGraph's public NCHW / KCRS and the
 * channels-last layout the contraction kernels consume.  `c_pad` >= C is the channel
 * count of the channels-last side (extra channels are written as zero / ignored).
 */
B200_API int b200_nchw_to_nhwc_u8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t c_pad, void* stream);
B200_API int b200_nhwc_to_nchw_u8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t c_pad, void* stream);

/* Channels-last [N,HW,C] -> [N,C,HW] for 4-byte elements (int32 / f32 outputs of the convolution). */
B200_API int b200_nhwc_to_nchw_b32(const void* in, void* out, int64_t N, int64_t C, int64_t HW, void* stream);

/*
 * One operand of op::v0::Concat (runtime/reference/concat.hpp): `rows` dense rows of row_bytes bytes written to rows
 * dst_pitch_bytes apart.  For axis a of a row-major tensor, rows = the product of the axes before a and row_bytes =
 * the operand's elements from axis a on; the caller offsets dst by the bytes of the operands already placed.
 */
B200_API int b200_copy_rows(const void* src, void* dst, int64_t rows, int64_t row_bytes, int64_t dst_pitch_bytes, void* stream);

/* Transpose a row-major [rows, cols] 1-byte matrix (B [K,N] of QuantizedDot -> W [N,K]). */
B200_API int b200_transpose_u8(const void* in, void* out, int64_t rows, int64_t cols, void* stream);

/*
 * MaxPool on channels-last u8 [N,H,W,C] -> [N,P,Q,C], C a multiple of 16.  Padding positions are
 * skipped as in runtime::reference::max_pool (src/ngraph/runtime/reference/max_pool.hpp:124-236).
 */
B200_API int b200_maxpool_nhwc_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C,
                                  int64_t win_h, int64_t win_w, int64_t stride_h, int64_t stride_w,
                                  int64_t pad_h, int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above,
                                  void* stream);
/* the same for i8 elements (padding positions are skipped; the lowest value is -128) */
B200_API int b200_maxpool_nhwc_i8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C,
                                  int64_t win_h, int64_t win_w, int64_t stride_h, int64_t stride_w,
                                  int64_t pad_h, int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above,
                                  void* stream);

/*
 * Global average pooling head on channels-last u8 [N,H,W,C] -> u8 [N,C]:
 *   Dequantize(scale_in, zp 0) -> AvgPool over the whole H x W window -> Quantize(scale_out, zp 0, RNE)
 * with the float sum taken sequentially in H,W order and one division by H*W, as
 * runtime::reference::avg_pool does for f32 (src/ngraph/runtime/reference/avg_pool.hpp:160-236).
 * (AvgPool directly on u8 accumulates in uint8 in the reference and wraps; the quantized graphs
 * therefore pool in f32, which is also where the CPU backend's fusion starts:
 * src/ngraph/runtime/cpu/pass/cpu_fusion.cpp:2160-2200.)  scale_in / scale_out: one float each, device memory.
 */
/*
 * Data dilation and negative padding of the convolutions, materialised on channels-last one-byte tensors (C a multiple of
 * 16): out [N, Ho, Wo, C] with Ho = (H - 1) * dilation_h + 1 - crop_h_below - crop_h_above (Wo alike) is the input with
 * dilation - 1 zero pixels between neighbours, less `crop` pixels at each border.  It stands for the data-dilation strides and
 * the negative part of padding_below / padding_above of op::v0::QuantizedConvolution and the fused convolutions
 * (src/ngraph/runtime/reference/convolution.hpp:59-265: CoordinateTransform with source dilation and signed padding, positions
 * that are not source coordinates are skipped); an ordinary convolution of the result with the non-negative part of the
 * padding then gives the reference's values.
 */
B200_API int b200_dilate_crop_nhwc_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C, int64_t dilation_h,
                                      int64_t dilation_w, int64_t crop_h_below, int64_t crop_w_below, int64_t crop_h_above,
                                      int64_t crop_w_above, void* stream);

B200_API int b200_global_avgpool_q_nhwc_u8(const void* in, void* out, const float* scale_in,
                                           const float* scale_out, int64_t N, int64_t H, int64_t W, int64_t C,
                                           void* stream);

/*
 * AvgPool with a window: replaces runtime::reference::avg_pool<T>
 * (src/ngraph/runtime/reference/avg_pool.hpp:160-236) as INTERPRETER dispatches it for op::v0::AvgPool
 * (src/ngraph/runtime/interpreter/int_executable.hpp, case AvgPool).  The window is walked in (h, w) order over the padded
 * image; image positions add their value, padding positions add 0 and count only with include_padding; the result is
 * sum / count with the sum taken sequentially in the element type.  P x Q is the op's output extent (in ceil mode it may
 * exceed the floor formula; positions beyond the padded image are not counted - the reference refuses such windows).
 * A geometry in which some window would count nothing returns B200_ERR_INVALID_ARGUMENT (the reference throws).
 *
 *   b200_avgpool_f32_nchw    f32 [N,C,H,W] -> f32 [N,C,P,Q]
 *   b200_avgpool_nhwc_bytes  the op applied to u8 / i8 directly, channels-last [N,H,W,C] -> [N,P,Q,C]: the reference keeps
 *                            the running sum in the one-byte type (it wraps modulo 256) and stores
 *                            nearbyint(float(sum) / count); reproduced literally
 *   b200_avgpool_q_nhwc      Dequantize(scale_in, zp 0) -> AvgPool(f32) -> Quantize(scale_out, zp 0, RNE) in one pass over
 *                            channels-last bytes (u8 or i8 on either side): the three ops' float operations in their order.
 *                            This is the graph CPUQuantFusion::construct_qavg_pool starts from
 *                            (src/ngraph/runtime/cpu/pass/cpu_fusion.cpp:2160-2200); scale_in / scale_out: one float each,
 *                            device memory.
 */
typedef struct b200_pool_params
{
    int64_t N, C, H, W;            /* input */
    int64_t P, Q;                  /* output extent */
    int64_t win_h, win_w, stride_h, stride_w;
    int64_t pad_h, pad_w;          /* padding below */
    int64_t pad_h_above, pad_w_above;
    int32_t include_padding;       /* include_padding_in_avg_computation */
} b200_pool_params;

B200_API int b200_avgpool_f32_nchw(const float* in, float* out, const b200_pool_params* geometry, void* stream);
B200_API int b200_avgpool_nhwc_bytes(const void* in, void* out, int type, const b200_pool_params* geometry, void* stream);
B200_API int b200_avgpool_q_nhwc(const void* in, int in_type, void* out, int out_type, const float* scale_in,
                                 const float* scale_out, const b200_pool_params* geometry, void* stream);

/*
 * Patch matrix for a convolution whose input has at most 4 channels (a network stem such as
 * 7x7 stride 2 on RGB): the tensor cores want 16-byte channel runs, which 3 channels cannot give.
 *   in  : channels-last u8 with exactly 4 channels per pixel [N,H,W,4] (see b200_nchw_to_nhwc_u8, c_pad 4)
 *   out : [N*P*Q, R*32] u8; row (n,p,q), segment r holds the 8 pixels w = q*stride_w - pad_w + 0..7 of input
 *         row h = p*stride_h - pad_h + r, 4 bytes each; taps s >= S and out-of-image pixels are zero.
 * b200_qgemm on this matrix with the filter packed the same way ([K, R*32]) is the convolution
 * (same accumulation as runtime::reference::general_convolution, src/ngraph/runtime/reference/convolution.hpp:59-265).
 * S <= 8, window dilation 1.
 */
B200_API int b200_im2col_c4_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t R, int64_t S,
                               int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                               int64_t pad_h_above, int64_t pad_w_above, void* stream);

/*
 * Constant weights in the layout the tensor cores read them in.  nGraph's CPU backend reorders constant weights into
 * DNNL's blocked formats (src/ngraph/runtime/cpu/pass/cpu_layout.cpp:531-720, ConvolutionLayout<QuantizedConvolution*>
 * inserting ConvertLayout nodes that constant folding then applies to the weights); this is the B200 counterpart.
 *   b200_packed_weights_bytes   size of the image of an [N, K] int8 matrix for k-blocks of bk (64 or 128) bytes
 *   b200_pack_weights_host      HOST function: row-major [N, K] -> image (done once, when the graph is compiled)
 *   b200_qconv_weight_block     the bk b200_qconv_packed expects for C input channels
 *   b200_qgemm_packed           b200_qgemm with packed_weights = image of W[N, K] for bk = 128
 *   b200_qconv_packed           b200_qconv with packed_filters = image of the [K, R*S*C] filter matrix (KRSC order)
 * Results are identical to the unpacked entry points; only the way weights reach shared memory differs (one bulk copy
 * per tile and k-block instead of one TMA box row per output channel).
 */
B200_API int64_t b200_packed_weights_bytes(int64_t N, int64_t K, int64_t bk);
B200_API int b200_pack_weights_host(const int8_t* w, int8_t* packed, int64_t N, int64_t K, int64_t bk);
B200_API int64_t b200_qconv_weight_block(int64_t C);
B200_API int b200_qgemm_packed(const void* A, int a_type, const int8_t* packed_weights, void* out, int64_t M, int64_t N,
                               int64_t K, const b200_epilogue* epilogue, void* stream);
B200_API int b200_qconv_packed(const void* data, int data_type, const int8_t* packed_filters, void* out,
                               const b200_conv_params* c, const b200_epilogue* epilogue, void* stream);

/*
 * Non-zero input / filter zero points for op::v0::QuantizedConvolution and op::v0::QuantizedDot
 * (src/ngraph/runtime/reference/convolution.hpp:236-258, dot.hpp:134-159): the reference multiplies (a - za) * (w - zw)
 * over the taps inside the image.  On the device the contraction runs on the stored bytes with the raw epilogue
 * (round_half_away == 2, int32 out) and one pass over those accumulators applies
 *     acc = S - zw * (input window sum) - za * (filter sum over the valid taps) + (valid taps) * C * za * zw
 * followed by the core requantisation (saturate((OUT)roundf((float)acc * scale[0]) + out_zero_point)).
 *   b200_strided_sums         out[o*n_inner + i] = sum_c x[o*outer_stride + i*inner_stride + c*sum_stride], x u8 or i8: the
 *                             filter's per-tap sums [K, R*S] from KCRS, the input's per-pixel channel sums [N, H*W] from
 *                             NCHW, the row sums of A / column sums of B of a matrix product
 *   b200_window_sums          per-pixel sums [N,H,W] -> per-output window sums [N,P,Q] (padding counts 0)
 *   b200_requant_zero_points  acc [N,P,Q,K] int32 -> out [N,P,Q,K] of e->out_type (U8, I8, I32); e must be a core epilogue
 *                             (round_half_away == 1, scale_count == 1).  filter_tap_sums [K,R,S] may be NULL when the
 *                             input zero point is 0, window_sums [N,P,Q] when the filter zero point is 0.
 * A matrix product [M,K] x [K,N] is the case N = 1, P = M, Q = 1, K = columns, H = M, W = 1, C = reduction length,
 * R = S = 1, strides and dilations 1, padding 0.
 */
typedef struct b200_zero_point_params
{
    int64_t N, P, Q, K; /* accumulator / output extents, K (output channels) fastest */
    int64_t H, W, C;    /* input image and channels per tap                          */
    int64_t R, S;       /* filter window                                             */
    int64_t stride_h, stride_w, dilation_h, dilation_w, pad_h, pad_w; /* padding below */
    int32_t input_zero_point, filter_zero_point;
} b200_zero_point_params;

B200_API int b200_strided_sums(const void* x, int x_type, int32_t* out, int64_t n_outer, int64_t n_inner, int64_t n_sum,
                               int64_t outer_stride, int64_t inner_stride, int64_t sum_stride, void* stream);
B200_API int b200_window_sums(const int32_t* pixel_sums, int32_t* out, const b200_zero_point_params* z, void* stream);
B200_API int b200_requant_zero_points(const int32_t* acc, const int32_t* filter_tap_sums, const int32_t* window_sums,
                                      const b200_zero_point_params* z, const b200_epilogue* e, void* out, void* stream);

/*
 * Stride-2 convolutions over <= 4 input channels (network stems, e.g. 7x7 stride 2 on RGB) on the tensor cores,
 * without a patch matrix: the NCHW input is regrouped into 2x2-pixel cells of 4 channels (16 bytes per cell, zero
 * outside the image); one output pixel then needs, per filter row pair, 4 neighbouring cells = 64 contiguous bytes.
 *   b200_stem_geometry          P, Q (output size), Hc, Wc (cell grid), Rc (cell rows per window); unsupported if a
 *                               filter row spans more than 4 cell columns (S > 7 or 8)
 *   b200_stem_pack_filter_host  HOST function: KCRS i8 filter -> [K, Rc*64] in the matching order (done once, at compile)
 *   b200_stem_cells_bytes       bytes the cell grid buffer must have: N*Hc*Wc*16 plus 2112 bytes the convolution may
 *                               read past the last cell (their contents do not matter and are never written)
 *   b200_stem_pack_input        device: NCHW one-byte input -> cell grid [N, Hc, Wc, 16]
 *   b200_stem_pack_input_f32    device: the same from the f32 input of a per-tensor op::v0::Quantize (scale[1], zero
 *                               point[1] of q_type u8 / i8, round_mode as in b200_quantize): Quantize fused into the packing
 *   b200_qconv_stem             the convolution with the fused epilogue; out is channels-last [N,P,Q,K]
 * Same accumulation as runtime::reference::general_convolution (src/ngraph/runtime/reference/convolution.hpp:59-265)
 * for strides {2,2}, window dilation 1; used for QuantizedConvolutionBias and friends like b200_qconv.
 */
B200_API int b200_stem_geometry(int64_t H, int64_t W, int64_t R, int64_t S, int64_t pad_h, int64_t pad_w,
                                int64_t pad_h_above, int64_t pad_w_above, int64_t* P, int64_t* Q, int64_t* Hc,
                                int64_t* Wc, int64_t* Rc);
B200_API int64_t b200_stem_cells_bytes(int64_t N, int64_t H, int64_t W, int64_t R, int64_t S, int64_t pad_h, int64_t pad_w,
                                       int64_t pad_h_above, int64_t pad_w_above);
B200_API int b200_stem_pack_filter_host(const int8_t* kcrs, int8_t* packed, int64_t K, int64_t C, int64_t R, int64_t S,
                                        int64_t pad_h, int64_t pad_w);
B200_API int b200_stem_pack_input(const void* in_nchw, void* cells, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t R, int64_t S, int64_t pad_h, int64_t pad_w, int64_t pad_h_above,
                                  int64_t pad_w_above, void* stream);
B200_API int b200_stem_pack_input_f32(const float* in_nchw, const float* scale, const void* zero_point, int q_type,
                                      int round_mode, void* cells, int64_t N, int64_t C, int64_t H, int64_t W, int64_t R,
                                      int64_t S, int64_t pad_h, int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above,
                                      void* stream);
B200_API int b200_qconv_stem(const void* cells, int data_type, const int8_t* packed_filters, void* out, int64_t N,
                             int64_t H, int64_t W, int64_t K, int64_t R, int64_t S, int64_t pad_h, int64_t pad_w,
                             int64_t pad_h_above, int64_t pad_w_above, const b200_epilogue* epilogue, void* stream);

/*
 * b200_stem_pack_input + b200_qconv_stem in one call that allocates nothing.  No counterpart in the reference: nGraph
 * backends allocate their workspaces when a Function is compiled.  The cell grid lives in a fixed 16 MiB device array
 * inside this library (b200_qconv_stem_static_capacity() bytes; a call needs b200_stem_cells_bytes(...) of it), looked up once per device at the first call on that device; that first call should be made before
 * a stream capture starts.  Larger problems are refused with B200_ERR_TOO_LARGE, and every other invalid argument (data
 * type, channel counts, epilogue record, null pointers) with its own code, before anything is launched, so a refused call
 * never writes the shared array.  The 16 MiB are part of the library's device image: every GPU context that loads the
 * library holds them until it exits, whether or not this entry point is ever called.  Nothing in
 * the array has to be zero beforehand: every cell, padding cells included, is written by the packing kernel before the
 * convolution reads it.  The array is shared by all callers of the device: two calls whose kernels can overlap in time
 * (different streams, different threads) race on it; calls on one stream are ordered and safe.  in_nchw is the one-byte
 * NCHW input [N, C <= 4, H, W]; the other arguments and the result are those of b200_qconv_stem.
 */
B200_API int64_t b200_qconv_stem_static_capacity(void);
B200_API int b200_qconv_stem_static(const void* in_nchw, int data_type, const int8_t* packed_filters, void* out, int64_t N,
                                    int64_t C, int64_t H, int64_t W, int64_t K, int64_t R, int64_t S, int64_t pad_h,
                                    int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above,
                                    const b200_epilogue* epilogue, void* stream);

/*
 * f32 glue operators: the float islands of a quantized graph (softmax, LayerNorm and GELU after
 * pass::FusedOpDecomposition, residual adds, dynamic activation scales), each with the arithmetic of the reference
 * kernel the INTERPRETER backend runs, so that results are identical and not merely close:
 *   b200_f32_binary      Add, Subtract, Multiply, Divide, Maximum, Minimum on equal shapes
 *                        (runtime/reference/add.hpp, subtract.hpp, multiply.hpp, divide.hpp, maximum.hpp, minimum.hpp)
 *   b200_f32_binary_periodic the same ops where one operand is a small tensor v that an op::v0::Broadcast would repeat along
 *                        new LEADING axes (a bias row added to every row, a scalar factor): out[i] = a[i] op v[i % period]
 *                        (v op a[i] with v_is_left), without the broadcast copy; n must be a multiple of period
 *   b200_f32_unary       Abs, Negative, Sqrt, Exp, Erf, Relu (abs.hpp, negate.hpp, sqrt.hpp, exp.hpp, erf.hpp, relu.hpp);
 *                        Exp and Erf are the double routine rounded to float
 *   b200_broadcast_b32   op::v0::Broadcast for 4-byte elements (broadcast.hpp): out_shape and the axes that are new
 *   b200_permute_b32     the axis permutation of a transposing op::v0::Reshape for 4-byte elements (reshape.hpp):
 *                        output axis i is input axis order[i]
 *   b200_reduce_f32      op::v0::Sum (Kahan-compensated, sum.hpp:56-90), op::v0::Max (max.hpp:32-58) and op::v0::Min (min.hpp) over an axis set,
 *                        inputs taken in row-major order like the reference
 *   b200_softmax_rows_f32 op::v0::Softmax over the last axis of a [rows, row_elements] matrix (softmax.hpp: max, exp(x - max),
 *                        Kahan sum, divide -- the same values as those five ops run one after another); rows longer
 *                        than 1535 elements return B200_ERR_UNSUPPORTED
 *   b200_layer_norm_rows_f32 op::v0::LayerNorm over the last axis with scale and bias (layer_norm.cpp:68-150): the values of
 *                        its decomposition (mean and variance through Kahan sums, sqrt(var + epsilon), divide, scale,
 *                        shift; every step rounded separately) from one kernel; rows longer than 1535 are unsupported
 *   b200_gelu_f32        op::v0::Gelu as its decomposition computes it (gelu.cpp:46-60): (0.5 * x) * (1 + erf(x / sqrt 2))
 *   b200_bmm_f32         op::v0::BatchMatMul / 2-D op::v0::Dot on f32 (batch_mat_mul.hpp, dot.hpp:108-160): a[b,M,K] x
 *                        b[b,K,N], the sum over k in double, in order, rounded to float once
 *   b200_gather_rows_b32 op::v0::Gather with axis 0 on a 2-D table of 4-byte elements and an i32 / i64 index vector
 *                        (gather.hpp); an index outside the table yields zeros (the reference does not check)
 */
typedef enum b200_f32_op
{
    B200_F32_ADD = 0,
    B200_F32_SUB = 1,
    B200_F32_MUL = 2,
    B200_F32_DIV = 3,
    B200_F32_MAX = 4,
    B200_F32_MIN = 5,
    B200_F32_ABS = 6,
    B200_F32_NEG = 7,
    B200_F32_SQRT = 8,
    B200_F32_EXP = 9,
    B200_F32_ERF = 10,
    B200_F32_RELU = 11
} b200_f32_op;

typedef enum b200_reduce_op
{
    B200_REDUCE_SUM = 0,
    B200_REDUCE_MAX = 1,
    B200_REDUCE_MIN = 2,
    B200_REDUCE_MAX_ABS = 3 /* Max over Abs(x): the two ops of a dynamic activation scale in one pass */
} b200_reduce_op;

B200_API int b200_f32_binary(int op, const float* a, const float* b, float* out, int64_t n, void* stream);
B200_API int b200_f32_binary_periodic(int op, const float* a, const float* v, float* out, int64_t n, int64_t period,
                                      int v_is_left, void* stream);
B200_API int b200_f32_unary(int op, const float* x, float* out, int64_t n, void* stream);
B200_API int b200_broadcast_b32(const void* in, void* out, const int64_t* out_shape, int rank, const int64_t* broadcast_axes,
                                int n_axes, void* stream);
B200_API int b200_permute_b32(const void* in, void* out, const int64_t* in_shape, int rank, const int64_t* order, void* stream);
B200_API int b200_reduce_f32(int op, const float* in, float* out, const int64_t* shape, int rank, const int64_t* axes,
                             int n_axes, void* stream);
B200_API int b200_softmax_rows_f32(const float* x, float* out, int64_t rows, int64_t row_elements, void* stream);
B200_API int b200_layer_norm_rows_f32(const float* x, const float* gamma, const float* beta, float* out, int64_t rows,
                                      int64_t row_elements, float epsilon, void* stream);
/* the same two kernels with the elementwise op that produced their input folded into the load: Softmax(x * *factor) for an
 * op::v1::Multiply by a broadcast scalar (factor: one element, device memory), LayerNorm(x + addend) for an op::v1::Add;
 * each product / sum is rounded once, exactly as the separate op would have stored it */
B200_API int b200_softmax_rows_scaled_f32(const float* x, const float* factor, float* out, int64_t rows, int64_t row_elements,
                                          void* stream);
B200_API int b200_layer_norm_rows_sum_f32(const float* x, const float* addend, const float* gamma, const float* beta, float* out,
                                          int64_t rows, int64_t row_elements, float epsilon, void* stream);
B200_API int b200_gelu_f32(const float* x, float* out, int64_t n, void* stream);
B200_API int b200_bmm_f32(const float* a, const float* b, float* out, int64_t batch, int64_t M, int64_t K, int64_t N,
                          void* stream);
B200_API int b200_gather_rows_b32(const void* table, int64_t n_rows, int64_t row_elements, const void* indices, int index_type,
                                  int64_t n_indices, void* out, void* stream);

/*
 * out[0] = input_scale[0] * filter_scale[0] / output_scale[0] in fp32, left to right: the requantisation
 * scale of op::v0::QuantizedDot / QuantizedConvolution (src/ngraph/runtime/reference/dot.hpp:154,
 * src/ngraph/runtime/reference/convolution.hpp:254) when the three scales are run-time tensors.
 */
B200_API int b200_requant_scale(const float* input_scale, const float* filter_scale, const float* output_scale,
                                float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_KERNELS_H */
