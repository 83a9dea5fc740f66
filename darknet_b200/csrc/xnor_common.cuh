// Shared helpers for the xnor_b200 kernels: error plumbing, geometry, launch-size helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "xnor_b200.h"

namespace xnor
{

// Last failing CUDA status seen by this library on the calling thread.
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e)
{
	g_last_cuda_error = (int)e;
	return XNOR_B200_ERR_CUDA;
}

// Checks the launch that was just issued.  cudaPeekAtLastError is legal under stream capture.
inline int check_launch()
{
	cudaError_t e = cudaPeekAtLastError();
	return e == cudaSuccess ? XNOR_B200_OK : cuda_fail(e);
}

// Number of SMs of the current device (cached per device index).
int sm_count();

inline int conv_out_dim(int in, int size, int stride, int pad) { return (in + 2 * pad - size) / stride + 1; }
inline int aligned_lda(int k) { return k + (256 - k % 256); }        // always adds, even when k%256==0
inline int aligned_n(int n) { return n + (32 - n % 32); }            // always adds, even when n%32==0
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int validate_desc(const xnor_b200_conv_desc * d);

// Process-wide overrides set through xnor_b200_set_tuning (all zero: every choice is the library's own).
const xnor_b200_tuning & tuning();

// Raises a kernel's dynamic shared-memory limit once per (device, kernel); later calls are a table lookup,
// so launchers stay free of runtime attribute calls once warmed up (e.g. while a stream is being captured).
int ensure_dynamic_smem(const void * kernel, size_t bytes);

// Internal launchers shared between translation units --------------------------------------

// A consumer of sign bits that the GEMM epilogue feeds directly: the packed activation operand (t_bit_input) of a
// following xnor layer with c % 32 == 0, stride 1.  Word (channel block, pixel) of this layer's output sign tensor is
// stored at every (row, K-word) of that operand where the consumer's im2col would have put it.
struct SinkParams
{
	uint32_t * operand;    // consumer's packed rows [image * n_out + row][ldw]
	int ldw;               // words per row
	int out_h, out_w;      // consumer's output map (= its input map: stride 1, "same" padding or 1x1)
	int n_out;
	int ks, pad, taps;
	int cb_offset;         // first 32-channel block of the consumer's input that this producer fills (route concat)
	int pool;              // 2: a 2x2 / stride-2 max-pool lies in between (OR of the four words); 0: none
	int up;                // 2: a nearest-neighbour x2 upsample lies in between; 1: none
	int win_w;             // consumer's rows are in 2x2-window-major order (out_w / 2), 0: row-major
};

// Optional extras of the integer GEMM.  win_w > 0: the columns of an image are this layer's pixels in
// 2x2-window-major order (index ((y/2)*win_w + x/2)*4 + (y%2)*2 + x%2), so four consecutive columns are one pool window.
struct GemmExtra
{
	int win_w;
	int out_w;
	int n_sinks;
	SinkParams sinks[2];
	// Short-K kernel only: build the B rows on the fly from x-packed sign planes [image][pl_c][pl_h][ceil(pl_w/32)]
	// (3x3, stride 1, pad 1 over pl_c channels, K order [c][ky][kx]) instead of reading a packed operand.
	const uint32_t * planes;
	int pl_c, pl_h, pl_w;
	// Same, from channel masks [image][pl_h][pl_w][pl_c/8] bytes (bit c%8 of byte c/8), pl_c 8 or 16, with the rows and the
	// weights in TAP-major K order (bit t*pl_c + c): a row is then nine neighbouring masks side by side.
	const uint8_t * masks;
	// Tensor-core kernel only, with a fused shortcut: also write the sign of shortcut_out as channel-packed words
	// [image][M/32][pixels per image] (the input_signs format of the layer that reads the sum).
	uint32_t * sum_signs;
	// ... or straight into the packed operand of a 1x1 / stride-1 xnor layer over exactly these filters: rows of sum_ldw words,
	// one row per pixel, word f/32 of a row = the signs of filters f .. f+31 at that pixel.
	uint32_t * sum_rows;
	int sum_ldw;
};

// True when launch_xnor_gemm would run such a layer on the short-K kernel, i.e. when `planes` may be used.
bool gemm_takes_planes(int M, int n_total, int c, int size, int stride, int pad);

#ifdef __CUDACC__
// Pixel (row-major index inside the image) of column `pixcol` of an image.
__device__ __forceinline__ int col_to_pixel(const GemmExtra & x, int pixcol)
{
	if (x.win_w == 0) { return pixcol; }
	const int q = pixcol >> 2;
	const int wy = q / x.win_w;
	const int wx = q - wy * x.win_w;
	return (2 * wy + ((pixcol >> 1) & 1)) * x.out_w + 2 * wx + (pixcol & 1);
}

// Stores sign word `word` of consumer-input pixel (iy, ix), channel block cb, at the place of the consumer's packed
// operand where its im2col puts tap (ky, kx): K-word cb*taps + ky*ks + kx of output pixel (iy + pad - ky, ix + pad - kx).
__device__ __forceinline__ void sink_store_tap(const SinkParams & s, int img, int iy, int ix, int cb, int tap, uint32_t word, int half = -1)
{
	const int ky = tap / s.ks;
	const int kx = tap - ky * s.ks;
	const int oy = iy + s.pad - ky;
	const int ox = ix + s.pad - kx;
	if (oy < 0 || oy >= s.out_h || ox < 0 || ox >= s.out_w) { return; }
	const size_t row = (s.win_w > 0) ? ((size_t)(oy >> 1) * s.win_w + (ox >> 1)) * 4 + (oy & 1) * 2 + (ox & 1)
	                                 : (size_t)oy * s.out_w + ox;
	uint32_t * dst = s.operand + ((size_t)img * s.n_out + row) * s.ldw + (size_t)(s.cb_offset + cb) * s.taps + tap;
	if (half < 0) { *dst = word; }
	else { reinterpret_cast<uint16_t *>(dst)[half] = (uint16_t)word; }      // a 16-filter tile owns one half of the word
}
#endif

// signs != nullptr: instead of C, only the sign bits of the output are written, 32 filters per word, laid out
// [image][M/32][pixel] (requires M % 32 == 0).
// GEMM with the batch folded into the column index: column j = b*n_per_image + p is written to
// C[(b*M + i)*ldc + p].  counts != nullptr selects the integer-accumulator output instead of C.
int launch_xnor_gemm(int M, int n_total, int n_per_image, int K,
		const uint32_t * A, int lda_words, const uint32_t * B, int ldb_words,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky,
		const float * shortcut_in, float * shortcut_out, int32_t * counts, cudaStream_t stream, uint32_t * signs = nullptr,
		const GemmExtra * extra = nullptr);

// Tensor-core (tcgen05, kind::i8 on bytes expanded in shared memory) variant of the same GEMM for large layers.
bool tc_gemm_eligible(int M, int n_total, int K);
int launch_xnor_gemm_tc(int M, int n_total, int n_per_image, int K,
		const uint32_t * A, int lda_words, const uint32_t * B, int ldb_words,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky,
		const float * shortcut_in, float * shortcut_out, int32_t * counts, cudaStream_t stream, uint32_t * signs = nullptr,
		const GemmExtra * extra = nullptr);
// Sticky device-side status (bounded wait expired in the tensor-core kernel); synchronous copy from the device.
int read_tc_error(int * out, bool clear);

// pool == nullptr: the tensor in memory is the convolution input; otherwise it is max-pooled on the fly.
// from_signs != 0: `input` is not fp32 but the sign words [image][c/32][in_h*in_w] left by a sign-only GEMM epilogue.
int launch_pack_input(const xnor_b200_conv_desc & d, const xnor_b200_pool_desc * pool, const float * input,
		uint32_t * t_bit_input, cudaStream_t stream, int from_signs = 0, int window_major = 0, uint32_t * words_scratch = nullptr);
// words_scratch != nullptr (pack_words_bytes(d) bytes, 16-byte aligned) lets large c%32==0 problems run as two passes.
size_t pack_words_bytes(const xnor_b200_conv_desc & d);

}  // namespace xnor
