/*
 * xnor_b200 -- C ABI of the B200 (sm_100a) XNOR-Net binarized-convolution forward path.
 *
 * Every entry point replaces one function (or one fused run of functions) of hank-ai/darknet's
 * xnor path; the comment above each declaration names the reference interface it stands in for
 * (file:line inside the darknet tree).  All pointers are DEVICE pointers unless a parameter
 * says "host".  `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 * No entry point synchronises, allocates or frees device memory unless its comment says so,
 * so every launch may be captured into a CUDA graph.
 *
 * Semantics are those of the reference's CPU bit path (the only one that is defined for every
 * layer shape): sign(v) = v > 0, out-of-image taps count as "not > 0", zero padding bits.
 * Bit i of a bit tensor lives in byte i/8 at position i%8.
 *
 * Return value: 0 on success, otherwise one of the XNOR_B200_ERR_* codes; nothing is launched
 * when an argument check fails.  There is no CPU fallback anywhere behind this interface.
 */
#ifndef XNOR_B200_H
#define XNOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported-symbol marker: the library is built with hidden visibility by default. */
#if defined(XNOR_B200_BUILD) && defined(__GNUC__)
#define XNOR_B200_API __attribute__((visibility("default")))
#else
#define XNOR_B200_API
#endif

#define XNOR_B200_OK               0
#define XNOR_B200_ERR_INVALID      1  /* a size, stride or enum argument is out of range            */
#define XNOR_B200_ERR_NULL         2  /* a required pointer is NULL                                */
#define XNOR_B200_ERR_SCRATCH      3  /* scratch buffer smaller than xnor_b200_scratch_bytes()     */
#define XNOR_B200_ERR_CUDA         4  /* a CUDA runtime call failed; see xnor_b200_last_cuda_error */
#define XNOR_B200_ERR_ALIGNMENT    5  /* a pointer or leading dimension is not aligned as required */
#define XNOR_B200_ERR_TOO_LARGE    6  /* a size exceeds a stated fixed limit of the entry point    */

#define XNOR_B200_LINEAR 0
#define XNOR_B200_LEAKY  1

/* Geometry of one [convolutional] xnor=1 layer: the fields of Darknet::Layer that the path reads
 * (src-lib/darknet_layers.hpp:39-78: batch, c, h, w, n, size, stride, pad, activation). */
typedef struct xnor_b200_conv_desc
{
	int batch;       /* images per call; the path computes ALL of them (the reference only image 0) */
	int c, h, w;     /* input channels, height, width (NCHW fp32)                                   */
	int n;           /* filters                                                                     */
	int size;        /* square kernel size                                                          */
	int stride;      /* stride_x == stride_y                                                        */
	int pad;         /* padding in pixels                                                           */
	int activation;  /* XNOR_B200_LINEAR or XNOR_B200_LEAKY (fused into the GEMM epilogue)          */
} xnor_b200_conv_desc;

/* Derived sizes, following make_convolutional_layer (src-lib/convolutional_layer.cpp:833-853)
 * and binary_align_weights (src-lib/convolutional_layer.cpp:1343-1351). */
typedef struct xnor_b200_conv_geom
{
	int out_h, out_w;
	int n_out;                 /* out_h*out_w, the GEMM N of one image                              */
	int k;                     /* size*size*c, the GEMM K in bits                                   */
	int new_lda;               /* k + (256 - k%256): bits per packed row of A and of B              */
	int bit_align;             /* n_out + (32 - n_out%32)                                           */
	int word_path;             /* 1 when c%32==0 (K ordered [c/32][tap][32]), else plain [c][tap]   */
	size_t weights_bytes;      /* n*new_lda/8: packed weights (the reference allocates one more)    */
	size_t packed_input_bytes; /* batch*n_out*new_lda/8: the packed, transposed B operand           */
	size_t output_floats;      /* batch*n*n_out                                                     */
} xnor_b200_conv_geom;

XNOR_B200_API const char * xnor_b200_strerror(int code);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread. */
XNOR_B200_API int xnor_b200_last_cuda_error(void);

/* Kernel-selection overrides for tests, benchmarks and tuning runs (no reference counterpart: Darknet has one kernel per
 * step).  Process-wide and read at every launch; set them while no other thread is launching.  A zeroed struct, or
 * xnor_b200_set_tuning(NULL), restores the library's own choices.  Every route computes identical results. */
#define XNOR_B200_ROUTE_AUTO    0  /* the library picks the GEMM kernel per call from its time estimates            */
#define XNOR_B200_ROUTE_INTEGER 1  /* integer-pipe kernels only (tiled, one-shot, short-row), tensor-core route off */
#define XNOR_B200_ROUTE_TENSOR  2  /* the tcgen05 kernel for every call                                            */
#define XNOR_B200_ROUTE_TILED   3  /* the tiled integer kernel for every call                                       */
typedef struct xnor_b200_tuning
{
	int gemm_route;           /* XNOR_B200_ROUTE_*                                                                     */
	int gemm_tile;            /* ROUTE_TILED only: 1-based tile configuration to pin (0 = estimated)                   */
	int gemm_split;           /* ROUTE_TILED only, with gemm_tile: cluster split-K factor 1..8 (0 = 1)                 */
	int pack_ctas_per_sm;     /* CTAs per SM the pack kernels size their grid for (0 = default)                        */
	int tc_kernel;            /* tcgen05 route: 0 = the library's choice, 1 = one tile per CTA, 2 = the persistent kernel         */
	int tc_wait_polls;        /* polls after which a barrier wait of the tcgen05 kernel gives up (0 = default limit)   */
	int tc_withhold_arrival;  /* failure-detection test aid: 1 = one producer arrival per tile is withheld, so that a  */
	                          /* bounded wait runs out and the kernel leaves through its give-up path                  */
	int pack_two_pass;        /* c%32==0 pack with room for sign words: 2 = sign words first, rows from the words; 0, 1 = one kernel */
} xnor_b200_tuning;
XNOR_B200_API int xnor_b200_set_tuning(const xnor_b200_tuning * tuning);

/* Fills *geom.  Replaces the size arithmetic of make_convolutional_layer
 * (src-lib/convolutional_layer.cpp:833-853) and binary_align_weights (:1343-1351). */
XNOR_B200_API int xnor_b200_conv_geometry(const xnor_b200_conv_desc * desc, xnor_b200_conv_geom * geom);

/* binarize_weights (src-lib/convolutional_layer.cpp:196-213) / fast_binarize_weights_gpu
 * (src-lib/convolutional_kernels.cu:116-132): per filter mean = (sequential fp32 sum of |w|)/size,
 * binary = w > 0 ? +mean : -mean.  weights, binary: [n][size] fp32; mean_arr: [n] (may be NULL).
 * The sum is taken in index order so the result equals the reference CPU value bit for bit. */
XNOR_B200_API int xnor_b200_binarize_weights(const float * weights, int n, int size, float * binary, float * mean_arr, void * stream);

/* binary_align_weights (src-lib/convolutional_layer.cpp:1339-1411) + get_mean_array (:131-140):
 * weights [n][c*size*size] fp32 (batch-norm already folded) -> align_bit_weights
 * (geom.weights_bytes bytes, row f at bit f*new_lda, K order per geom.word_path, zero padding)
 * and mean_arr [n].  invert != 0 complements every byte when c%32==0, the layout the reference
 * stores in GPU builds (:1395-1401); the GEMM below expects invert == 0.  Load-time step. */
XNOR_B200_API int xnor_b200_binary_align_weights(const xnor_b200_conv_desc * desc, const float * weights,
		uint8_t * align_bit_weights, float * mean_arr, int invert, void * stream);

/* float_to_bit (src-lib/gemm.cpp:1510-1534) / float_to_bit_gpu (src-lib/im2col_kernels.cu:310-317):
 * bit i of dst = src[i] > 0.  dst receives ceil(size/32)*4 bytes and must be 4-byte aligned. */
XNOR_B200_API int xnor_b200_float_to_bit(const float * src, uint8_t * dst, size_t size, void * stream);

/* repack_input + float_to_bit (src-lib/gemm.cpp:2202-2220, :1510) / repack_input_gpu_bin
 * (src-lib/im2col_kernels.cu:715-724): input [c][h*w] fp32 -> packed [c/32][h*w] uint32,
 * bit (ch%32) = input > 0.  Requires c%32 == 0. */
XNOR_B200_API int xnor_b200_repack_input_bin(const float * input, uint32_t * packed, int w, int h, int c, void * stream);

/* The whole input-side chain in one kernel, no float im2col buffer:
 *   c%32==0: repack_input_gpu_bin -> im2col_ongpu -> transpose_uint32_gpu
 *            (src-lib/convolutional_kernels.cu:220-231; CPU src-lib/convolutional_layer.cpp:1475-1517)
 *   else:    im2col_align_ongpu -> float_to_bit_gpu -> transpose_bin_gpu
 *            (src-lib/convolutional_kernels.cu:236-245; CPU im2col_cpu_custom_bin + transpose_bin,
 *            src-lib/convolutional_layer.cpp:1534-1541)
 * input [batch][c][h][w] fp32 -> t_bit_input [batch*n_out][new_lda/8] bytes: row (b*n_out + p) holds
 * the K sign bits of output pixel p of image b followed by zero padding (the reference leaves that
 * padding unwritten on the GPU).  t_bit_input must be 16-byte aligned. */
XNOR_B200_API int xnor_b200_pack_input(const xnor_b200_conv_desc * desc, const float * input, uint8_t * t_bit_input, void * stream);

/* The same packing in two passes for c%32==0, the reference's own split (repack_input_gpu_bin first,
 * src-lib/im2col_kernels.cu:715-724, then im2col + transpose on the words): pass one streams the fp32 input once
 * and leaves `words` = uint32 [batch][c/32][h*w] (xnor_b200_pack_words_bytes(desc) bytes, 16-byte aligned), pass two
 * builds t_bit_input from those.  Taken only while xnor_b200_tuning.pack_two_pass is 2 (otherwise the call is
 * xnor_b200_pack_input); the single kernel is as fast or faster on every shape measured, so this is kept for callers
 * that want the channel-packed words as a by-product.  xnor_b200_conv_forward does the same when its scratch buffer
 * has xnor_b200_pack_words_bytes() bytes more than xnor_b200_scratch_bytes() and the tuning asks for it. */
XNOR_B200_API size_t xnor_b200_pack_words_bytes(const xnor_b200_conv_desc * desc);
XNOR_B200_API int xnor_b200_pack_input_staged(const xnor_b200_conv_desc * desc, const float * input, uint32_t * words,
		uint8_t * t_bit_input, void * stream);

/* gemm_nn_custom_bin_mean_transposed_gpu (src-lib/im2col_kernels.cu:1156-1193), CPU
 * gemm_nn_custom_bin_mean_transposed (src-lib/gemm.cpp:907-1019) + add_bias
 * (src-lib/convolutional_layer.cpp:1269-1289) + leaky (src-lib/gemm.cpp:1472-1498):
 *   count = #agreeing bits of A row i and B row j among the first K;
 *   C[i*ldc + j] = act( fl( fl((2*count - K) * mean_arr[i]) + bias[i] ) );
 *   if shortcut_out: shortcut_out[i*ldc + j] = shortcut_in[i*ldc + j] + C[i*ldc + j].
 * A: M rows of lda bits, B: N rows of ldb bits, both with ZERO padding bits beyond K (A is NOT
 * inverted).  lda, ldb multiples of 128 and >= K; A, B 16-byte aligned.  bias, shortcut_* may be NULL. */
XNOR_B200_API int xnor_b200_gemm_bin_mean_transposed(int M, int N, int K,
		const uint8_t * A, int lda, const uint8_t * B, int ldb,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky_activation,
		const float * shortcut_in, float * shortcut_out, void * stream);

/* The integer accumulators of the GEMM above, for bit-exact checks: counts[i*N + j] = number of
 * agreeing bits among the first K -- the reference's `count` after `count - f1`
 * (src-lib/gemm.cpp:964-970, src-lib/im2col_kernels.cu:930-936). */
XNOR_B200_API int xnor_b200_gemm_counts(int M, int N, int K, const uint8_t * A, int lda, const uint8_t * B, int ldb,
		int32_t * counts, void * stream);

/* Diagnostics (no reference counterpart; Darknet aborts on any CUDA error instead).  The tensor-core GEMM
 * bounds every wait on a shared-memory barrier; if a wait ever runs out, the kernel skips its remaining work,
 * releases its tensor memory and sets a sticky device-side status word.  This call synchronises the device,
 * stores that word in *status (0 = nothing happened) and clears it. */
XNOR_B200_API int xnor_b200_take_device_status(int * status);

/* Bytes of scratch xnor_b200_conv_forward needs (= geom.packed_input_bytes, 256-byte rounded).  The
 * reference sizes net.workspace from other layers and over-allocates two bit_align*K*4-byte buffers
 * per layer (src-lib/convolutional_layer.cpp:1413-1418); this path owns its scratch explicitly. */
XNOR_B200_API size_t xnor_b200_scratch_bytes(const xnor_b200_conv_desc * desc);

/* The xnor branch of forward_convolutional_layer_gpu (src-lib/convolutional_kernels.cu:204-262) for the
 * whole batch: pack_input into scratch, then the GEMM with the batch folded into N and the epilogue
 * writing NCHW output [batch][n][out_h*out_w].  align_bit_weights / mean_arr come from
 * xnor_b200_binary_align_weights(invert = 0); biases [n]; shortcut_in/out [batch][n][n_out] or NULL
 * (the fused [shortcut] of src-lib/darknet_network.cpp:1799-1813).  scratch 256-byte aligned. */
XNOR_B200_API int xnor_b200_conv_forward(const xnor_b200_conv_desc * desc, const float * input,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		float * output, const float * shortcut_in, float * shortcut_out,
		void * scratch, size_t scratch_bytes, void * stream);

/* A [maxpool] layer placed directly in front of an xnor convolution (fields of src-lib/maxpool_layer.cpp:85-135:
 * size, stride, padding; in_h/in_w = the maxpool's input, i.e. the tensor that is actually in memory).  The
 * convolution descriptor passed with it describes the POOLED tensor: desc.h = (in_h + pad - size)/stride + 1. */
typedef struct xnor_b200_pool_desc
{
	int size, stride, pad;
	int in_h, in_w;
} xnor_b200_pool_desc;

/* forward_maxpool_layer_gpu (src-lib/maxpool_layer_kernels.cu:48-86, :107-167) followed by the input-side chain
 * of xnor_b200_pack_input, in one kernel: the next layer only needs sign(max(window)), which is the OR of the
 * signs of the in-image window elements, so the pooled tensor is never written or re-read.  Output identical
 * to xnor_b200_pack_input applied to the maxpool output. */
XNOR_B200_API int xnor_b200_pack_input_pooled(const xnor_b200_conv_desc * desc, const xnor_b200_pool_desc * pool,
		const float * input, uint8_t * t_bit_input, void * stream);

/* xnor_b200_conv_forward with the preceding [maxpool] folded into the pack kernel (see above).  Usable when
 * nothing but this convolution reads the maxpool output (the chains conv -> maxpool -> xnor conv of the tiny
 * networks). */
XNOR_B200_API int xnor_b200_conv_forward_pooled(const xnor_b200_conv_desc * desc, const xnor_b200_pool_desc * pool,
		const float * input, const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		float * output, const float * shortcut_in, float * shortcut_out,
		void * scratch, size_t scratch_bytes, void * stream);

/* Operands of xnor_b200_conv_forward_io.  Exactly one of input / input_signs / input_packed is given; at least one
 * of output, output_signs and sinks, and not both output and output_signs.
 *   input_signs   the previous xnor layer's output as sign bits, 32 channels per word, [batch][c/32][h*w] (with
 *                 `pool`: [batch][c/32][in_h*in_w] of the tensor in front of the maxpool) when c % 32 == 0;
 *                 when c % 32 != 0 (the first xnor layer behind a float convolution): x-packed sign planes
 *                 [batch][c][h][ceil(w/32)], bit x%32 of word x/32 = "value at column x > 0", no `pool`
 *                 (xnor_b200_float_conv3_io writes them already pooled)
 *   output_signs  this layer's output as sign bits only, [batch][n/32][out_h*out_w]; needs n % 32 == 0 and no
 *                 shortcut; the activation plays no role (leaky keeps the sign) */
/* A following xnor layer that this layer feeds directly: the GEMM epilogue stores every 32-filter sign word at each
 * place of the consumer's packed activation operand (its scratch buffer) where the consumer's own im2col + bit-pack
 * would have put it, so the consumer needs no pack kernel, and a [maxpool] size 2 / stride 2, an [upsample] stride 2
 * or a [route] concatenation between the two layers needs no kernel either.  The consumer must have c % 32 == 0,
 * stride 1 and size 3 / pad 1 or size 1 / pad 0, and the same batch.  consumer_scratch must have been zero-filled once
 * (cudaMemset) before the first forward and be written by nothing else: padding taps and the alignment tail of every
 * row are the zeros nobody ever overwrites. */
typedef struct xnor_b200_sign_sink
{
	const xnor_b200_conv_desc * consumer;
	void * consumer_scratch;       /* the scratch the consumer is later run with (input_packed = 1) */
	int channel_offset;            /* first input channel of the consumer that this layer provides (multiple of 32) */
	int pool;                      /* 2: a 2x2 / stride-2 max-pool lies in between (this layer then needs window_major = 1); 0: none */
	int upsample;                  /* 2: a nearest-neighbour x2 upsample lies in between; 0 or 1: none */
	int consumer_window_major;     /* the consumer is run with window_major = 1 */
} xnor_b200_sign_sink;

typedef struct xnor_b200_conv_io
{
	const float * input;
	const uint32_t * input_signs;
	const xnor_b200_pool_desc * pool;     /* optional maxpool between the previous layer and this one */
	float * output;                       /* may be NULL together with shortcut_out: only the fused sum is written then */
	uint32_t * output_signs;
	const float * shortcut_in;
	float * shortcut_out;
	int input_packed;                     /* 1: the producers' sinks have already filled this layer's scratch; no input pointer */
	int window_major;                     /* 1: the rows of this layer's packed operand (= the columns of its GEMM) are its output
	                                         pixels in 2x2-window-major order, ((y/2)*(w/2) + x/2)*4 + (y%2)*2 + x%2, so that a
	                                         pooled sink finds each window in four consecutive columns; outputs are unaffected */
	const xnor_b200_sign_sink * sinks;    /* up to 2 direct consumers; may be combined with `output` (fp32 for a [route]) */
	int n_sinks;
	const uint8_t * input_masks;          /* fourth kind of input, for the first xnor layer behind xnor_b200_float_conv3_io when
	                                         xnor_b200_conv_takes_masks() says so: channel masks [batch][h][w][c/8] (bit c%8 of byte
	                                         c/8 = "channel c > 0").  The GEMM then builds its rows itself, in TAP-major K order, so
	                                         the weights argument must be the xnor_b200_tap_major_weights() copy: */
	int tap_major_weights;                /* 1 = it is; input_masks is refused otherwise */
	uint32_t * shortcut_signs;            /* optional, with shortcut_out (n % 32 == 0): the sign of the fused sum as channel-packed
	                                         words [batch][n/32][out_h*out_w], i.e. the input_signs of the xnor layer that reads the
	                                         [shortcut]; that layer then packs from 1 bit per value instead of the fp32 sum.  The call
	                                         runs on the tensor-core kernel whatever its size, so use it for batched layers */
	const xnor_b200_sign_sink * shortcut_sink;  /* optional, same conditions: when the reader of the [shortcut] is a 1x1 / stride-1 /
	                                         pad-0 xnor layer over exactly these n channels on the same map, the signs of the sum go
	                                         straight into its packed operand (consumer_scratch, zero-filled once at load time); it
	                                         then runs with input_packed = 1 and no pack kernel.  channel_offset, pool, upsample and
	                                         consumer_window_major of the sink must be 0 */
} xnor_b200_conv_io;

/* 1 when a layer can take input_masks: c is 8 or 16, size 3, stride 1, pad 1 (and no route pinned through xnor_b200_set_tuning). */
XNOR_B200_API int xnor_b200_conv_takes_masks(const xnor_b200_conv_desc * desc);

/* Re-orders packed weights of a c % 32 != 0 layer from the reference's K order (bit c*size*size + tap,
 * src-lib/convolutional_layer.cpp:1403-1411) to tap-major (bit tap*c + c'), same row pitch.  XNOR-popcount does not care
 * about the order as long as both operands agree; tap-major makes an activation row nine neighbouring channel masks. */
XNOR_B200_API int xnor_b200_tap_major_weights(const xnor_b200_conv_desc * desc, const uint8_t * align_bit_weights, uint8_t * tap_major,
		void * stream);

/* xnor_b200_conv_forward for chains of xnor layers.  A layer marked bin_output=1 feeds nothing but the next
 * binarised convolution (src-lib/darknet_network.cpp:1794-1797 drops its activation for that reason), which only
 * looks at the sign of every value: with output_signs the GEMM epilogue writes that sign, 1 bit per value, instead
 * of the fp32 tensor, and the next layer's pack kernel reads the words (ORing them over the pool window when a
 * [maxpool] sits in between, src-lib/maxpool_layer_kernels.cu:48-86).  The bits equal what the next layer would
 * have derived from the fp32 tensor, so every later result is unchanged bit for bit. */
XNOR_B200_API int xnor_b200_conv_forward_io(const xnor_b200_conv_desc * desc, const xnor_b200_conv_io * io,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		void * scratch, size_t scratch_bytes, void * stream);

/* The float convolution in front of the path (3 input channels -> 16/32 filters in the xnor networks): the float
 * branch of forward_convolutional_layer_gpu (src-lib/convolutional_kernels.cu:373-434, cuDNN or im2col + sgemm) +
 * add_bias_gpu + leaky activate_array_ongpu (src-lib/activation_kernels.cu:34) as one direct-convolution kernel
 * for layers with c*size*size <= 128.  weights [n][c*size*size] (batch-norm folded), biases [n] or NULL,
 * output [batch][n][out_h*out_w].  fp32 throughout; sums run over (channel, ky, kx) with fused multiply-adds, so
 * results agree with cuDNN to rounding (about 1e-6 relative), not bit for bit. */
XNOR_B200_API int xnor_b200_float_conv_small(const xnor_b200_conv_desc * desc, const float * input, const float * weights,
		const float * biases, float * output, void * stream);

/* The same first float layer when it has 3 input channels, size 3, stride 1, pad 1 (all xnor networks), computed as
 * 2x2 output blocks per thread, optionally with the [maxpool] size 2 / stride 2 that follows it applied in registers
 * (pool = 2, needs even h and w; pool = 0: none), and optionally reduced to what a following xnor layer reads:
 *   output              fp32 [batch][n][h][w] (pool 0) or [batch][n][h/2][w/2] (pool 2), bias and activation applied
 *   output_sign_planes  pool 2 only: sign of the pooled output as x-packed planes [batch][n][h/2][ceil(w/2/32)],
 *                       the input_signs format of xnor_b200_conv_forward_io for c % 32 != 0
 *   output_sign_masks   the signs channel-packed per pixel, [batch][h/2][w/2][ceil(n/8)] bytes (pool 2: the input_masks
 *                       format of xnor_b200_conv_forward_io) or [batch][h][w][ceil(n/8)] bytes (pool 0; with n = 32 the four
 *                       bytes of a pixel are one word of the input_signs format, [batch][1][h*w], for an xnor layer over
 *                       those 32 channels, e.g. the stride-2 layer behind darknet53's first convolution)
 * Exactly one of the three is non-NULL.  Every value is formed as in xnor_b200_float_conv_small, so the planes equal
 * the sign of maxpool(that call's output) bit for bit.  Replaces forward_convolutional_layer_gpu (float branch) +
 * forward_maxpool_layer_gpu (src-lib/maxpool_layer_kernels.cu:48-86) + the sign step of the next layer. */
XNOR_B200_API int xnor_b200_float_conv3_io(const xnor_b200_conv_desc * desc, int pool, const float * input, const float * weights,
		const float * biases, float * output, uint32_t * output_sign_planes, uint8_t * output_sign_masks, void * stream);

/* The float convolutions behind the path (many channels on a small map: the 3x3 256->512 layer on 13x13 and the
 * 1x1 layers in front of the yolo heads): the same float branch of forward_convolutional_layer_gpu
 * (src-lib/convolutional_kernels.cu:373-434) + add_bias_gpu + activate_array_ongpu, for stride 1 and either
 * size 3 / pad 1 (c % 8 == 0, (h+2)*(w+2) <= 1024) or size 1 / pad 0 (c % 32 == 0).  The channels are split over a
 * thread-block cluster so that a batch-1 layer still covers the chip; partial sums are added in a fixed order.
 * Weights are re-blocked once at load time: _weights_bytes gives the size of the blocked copy (0 for a shape the
 * kernel does not take), _prepare fills it from Darknet's [n][c*size*size] weights (batch-norm folded), and the
 * forward takes the blocked copy (16-byte aligned).  Results agree with cuDNN to rounding, not bit for bit. */
XNOR_B200_API size_t xnor_b200_float_conv_map_weights_bytes(const xnor_b200_conv_desc * desc);
XNOR_B200_API int xnor_b200_float_conv_map_prepare(const xnor_b200_conv_desc * desc, const float * weights, float * blocked, void * stream);
XNOR_B200_API int xnor_b200_float_conv_map(const xnor_b200_conv_desc * desc, const float * input, const float * blocked_weights,
		const float * biases, float * output, void * stream);
/* 1x1 / stride-1 / pad-0 float convolutions with many pixels (the same layers at batch: tens of thousands of pixels, where
 * the cluster split above no longer pays): one GEMM over all images on the tensor cores at fp32 accuracy -- every operand is
 * split into a tf32 head and a tf32 remainder and three tcgen05.mma kind::tf32 products are accumulated per pair -- with
 * add_bias_gpu and the linear / leaky activation in the epilogue.  weights: Darknet's [n][c] (batch-norm folded), any c and n.
 * Replaces the per-image cuBLAS call of the float branch (src-lib/convolutional_kernels.cu:373-434).  Agrees with an fp64
 * convolution to fp32 rounding (a few 1e-7 relative), not with cuBLAS bit for bit. */
XNOR_B200_API int xnor_b200_float_conv_1x1_tc(const xnor_b200_conv_desc * desc, const float * input, const float * weights,
		const float * biases, float * output, void * stream);
/* Same, for the convolution right in front of a [yolo] layer: yolo_entries = 4 + 1 + classes (n must be a multiple of
 * it) also applies that layer's activation step (xnor_b200_yolo_activate below) to the result; 0 = plain call. */
XNOR_B200_API int xnor_b200_float_conv_map_yolo(const xnor_b200_conv_desc * desc, const float * input, const float * blocked_weights,
		const float * biases, float * output, int yolo_entries, void * stream);

/* The activation step of forward_yolo_layer_gpu (src-lib/yolo_layer.cpp:1439-1489) behind the path: logistic on the
 * x, y, objectness and class entries of every anchor, w and h raw, in one pass.  input/output
 * [batch][anchors][4 + 1 + classes][hw] (may be the same pointer).  Box decoding and NMS: xnor_b200_yolo_detections below. */
XNOR_B200_API int xnor_b200_yolo_activate(const float * input, float * output, int batch, int anchors, int classes, int hw, void * stream);
/* The activation step of the [region] head (forward_region_layer, src-lib/region_layer.cpp:494-537): logistic on x, y and
 * objectness, w and h raw, and with softmax != 0 a softmax over the class entries of every anchor and cell.
 * input/output [batch][anchors][coords + 1 + classes][hw], different pointers.  Agrees with Darknet's softmax to rounding. */
XNOR_B200_API int xnor_b200_region_activate(const float * input, float * output, int batch, int anchors, int coords, int classes,
		int softmax, int hw, void * stream);

/* ---- detection heads on the device ------------------------------------------------------------------------------
 * Darknet pulls every [yolo] output to the host after each forward (src-lib/yolo_layer.cpp:1439-1489) and decodes, filters
 * and suppresses there.  These three calls do it on the device and leave a compact list of rows to copy back. */
#define XNOR_B200_MAX_DETECTIONS 4096          /* largest max_dets (the suppression kernel keeps its lists in shared memory) */

/* One [yolo] layer after its activation step (xnor_b200_yolo_activate): output [batch][n][4 + 1 + classes][h * w];
 * anchors = the layer's own n anchor boxes in network pixels, {w0, h0, w1, h1, ...} = biases[2*mask[a]], biases[2*mask[a]+1]
 * (src-lib/yolo_layer.cpp:22-42); new_coords as in the cfg. */
typedef struct xnor_b200_yolo_head
{
	const float * output;
	int w, h, n, classes;
	float anchors[32];
	int new_coords;
} xnor_b200_yolo_head;

/* Device buffers of a detection list, one list per image: boxes [batch][max_dets][4] = {x, y, w, h} (16-byte aligned),
 * objectness [batch][max_dets], probs [batch][max_dets][classes], count [batch].  count may exceed max_dets when more
 * detections pass the threshold than fit; only the first max_dets are stored, in the reference's scan order. */
typedef struct xnor_b200_detections
{
	float * boxes;
	float * objectness;
	float * probs;
	int * count;
	int max_dets;
	int classes;
} xnor_b200_detections;

/* get_yolo_detections + get_yolo_box + correct_yolo_boxes (src-lib/yolo_layer.cpp:1306-1348, :22-42, :1161-1222) for every
 * image of the batch: each (cell, anchor) with objectness > thresh becomes a detection with prob[j] = objectness *
 * class probability where that exceeds thresh, else 0.  img_w, img_h, relative, letter as in get_network_boxes
 * (src-lib/darknet_network.cpp:1250).  append = 0 starts the lists, append = 1 continues them behind what an earlier head
 * left (a network's heads in layer order, as fill_network_boxes does). */
XNOR_B200_API int xnor_b200_yolo_detections(const xnor_b200_yolo_head * head, int batch, int netw, int neth, int img_w, int img_h,
		float thresh, int relative, int letter, int append, const xnor_b200_detections * dets, void * stream);

/* do_nms_sort (src-lib/box.cpp:951-1003): per class, in decreasing order of that class's probability, a kept detection
 * zeroes the class probability of every later detection whose box_iou (:310-344) with it exceeds nms_thresh.  Equal
 * probabilities keep their storage order (the reference's std::sort leaves that order unspecified). */
XNOR_B200_API int xnor_b200_nms_sort(const xnor_b200_detections * dets, int batch, float nms_thresh, void * stream);

/* The (detection, class) pairs with a probability above zero, detection-major, as rows of 7 floats {x, y, w, h, objectness,
 * class, probability}: rows [batch][max_rows][7], row_count [batch] (may exceed max_rows; the surplus is not stored). */
XNOR_B200_API int xnor_b200_detection_rows(const xnor_b200_detections * dets, int batch, float * rows, int max_rows, int * row_count,
		void * stream);

/* Bytes of the library-resident scratch array behind xnor_b200_conv_forward_static. */
#define XNOR_B200_STATIC_SCRATCH_BYTES (8u << 20)

/* xnor_b200_conv_forward for callers that cannot allocate device memory or pass a scratch buffer (a plugin
 * slot that is handed nothing but layer inputs and outputs, a server whose memory pool is sealed after
 * start-up, a real-time loop in which cudaMalloc's implicit synchronisation is not acceptable).  It has no
 * counterpart in the reference, whose layers always borrow net.workspace.  Same arguments and results as
 * xnor_b200_conv_forward, minus scratch: the packed activation operand goes into a fixed
 * XNOR_B200_STATIC_SCRATCH_BYTES array that is part of the library image (every GPU that loads the library
 * holds those bytes until the process exits).  The call makes no cudaMalloc/cudaFree and uses no allocating
 * library routine.
 *   - Limit: returns XNOR_B200_ERR_TOO_LARGE when geom.packed_input_bytes (batch*n_out*new_lda/8) exceeds
 *     XNOR_B200_STATIC_SCRATCH_BYTES; nothing is launched in that case.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current) and remembers it; make that first call before starting any stream capture.  Under the CUDA
 *     runtime's lazy module loading that first call is also where the 8 MiB array is materialised on the device, so
 *     it is the one call of this entry point that may allocate inside the driver: make it at start-up.
 *   - All calls on one device share the one array and it keeps the previous call's contents.  Nothing in it
 *     needs clearing (each call rewrites every word it later reads), but two calls whose kernels can overlap
 *     on the GPU -- different streams, or graph branches -- race on it: serialise them. */
XNOR_B200_API int xnor_b200_conv_forward_static(const xnor_b200_conv_desc * desc, const float * input,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		float * output, const float * shortcut_in, float * shortcut_out, void * stream);

/* Measurement helpers (no reference counterpart: the reference ships no peak figures).  Each runs a
 * register-resident loop on every SM, synchronises, and returns giga binary-ops per second
 * (64 per 32-bit XOR+POPC+ADD; 2*16*8*256 per b1 mma) in *gops, with the elapsed milliseconds in *ms.
 * These two calls synchronise the device. */
XNOR_B200_API int xnor_b200_measure_popc_peak(int iters, double * gops, double * ms);
XNOR_B200_API int xnor_b200_measure_bmma_peak(int iters, double * gops, double * ms);
/* Same, for the tensor-core route: back-to-back tcgen05.mma kind::i8 (M=128, N=256, K=32) from resident
 * shared-memory tiles on every SM, counted as 2*M*N*K operations per MMA (the GEMM's own convention). */
XNOR_B200_API int xnor_b200_measure_umma_i8_peak(int iters, double * gops, double * ms);
/* Same for tcgen05.mma kind::mxf4 (M=128, N=256, K=64, 4-bit operands, scale factors 2^0), the instruction of the one-tile
 * tensor-core kernel. */
XNOR_B200_API int xnor_b200_measure_umma_mxf4_peak(int iters, double * gops, double * ms);

#ifdef __cplusplus
}
#endif
#endif /* XNOR_B200_H */
