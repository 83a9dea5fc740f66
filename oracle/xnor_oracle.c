/*
 * TEST INFRASTRUCTURE -- CPU oracle for the XNOR-Net binarized-convolution forward path.
 *
 * A plain-C restatement of the reference's CPU algorithm (hank-ai/darknet), one function per
 * reference function, each citing the reference file:line it follows.  It exists so that the
 * CUDA path can be checked bit-for-bit on machines where the reference tree is not present.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may load this library; the
 * product library never links, loads or falls back to it.
 *
 * Parity pin: the reference ships no golden vectors or tests for this path.  This restatement
 * is pinned against the reference's own functions compiled unmodified (oracle/_ref, built by
 * the Makefile beside this file) and against fixtures generated from that build
 * (tests/golden/).  Where the reference CPU code is undefined (1x1 or strided layers whose
 * channel count is not a multiple of 32, batch > 1) this file is the closed-form definition:
 *     out[f][p] = act( fl( fl( (2*cnt - K) * mean_f ) + bias_f ) ),
 *     cnt = #{ k : (w_fk > 0) == (x_pk > 0) },  padded taps count as "not > 0".
 *
 * Bit conventions: bit i of a bit array lives in byte i/8 at position i%8 (LSB first),
 * as src-lib/gemm.hpp:12-20 (set_bit/get_bit) and src-lib/gemm.cpp:1510-1534 (float_to_bit).
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ---- geometry ------------------------------------------------------------------------- */

/* src-lib/convolutional_layer.cpp convolutional_out_height/width: (in + 2*pad - size)/stride + 1 */
ORACLE_API int oracle_out_dim(int in, int size, int stride, int pad)
{
	return (in + 2 * pad - size) / stride + 1;
}

/* src-lib/convolutional_layer.cpp:1345 and :848-851 -- always adds, even when k % 256 == 0 */
ORACLE_API int oracle_new_lda(int k)
{
	return k + (256 - k % 256);
}

/* src-lib/convolutional_layer.cpp:838-840 -- always adds, even when n % 32 == 0 */
ORACLE_API int oracle_bit_align(int n)
{
	return n + (32 - n % 32);
}

static inline void put_bit(uint8_t * dst, size_t i) { dst[i / 8] |= (uint8_t)(1u << (i % 8)); }
static inline int  read_bit(const uint8_t * src, size_t i) { return (src[i / 8] >> (i % 8)) & 1; }

/* ---- a1: binarize_weights, src-lib/convolutional_layer.cpp:196-213 --------------------- */
/* mean = (sequential fp32 sum of |w|) / size ; binary = w > 0 ? +mean : -mean */
ORACLE_API void oracle_binarize_weights(const float * weights, int n, int size, float * binary)
{
	for (int f = 0; f < n; ++f)
	{
		volatile float mean = 0.0f; /* volatile: forbid re-association / wider accumulation */
		for (int i = 0; i < size; ++i)
		{
			mean = mean + fabsf(weights[(size_t)f * size + i]);
		}
		float m = mean / (float)size;
		for (int i = 0; i < size; ++i)
		{
			binary[(size_t)f * size + i] = (weights[(size_t)f * size + i] > 0) ? m : -m;
		}
	}
}

/* ---- a3: float_to_bit, src-lib/gemm.cpp:1510-1534 -------------------------------------- */
/* dst must hold size/8 + 1 bytes; all of them are written (zero beyond the last bit). */
ORACLE_API void oracle_float_to_bit(const float * src, uint8_t * dst, size_t size)
{
	memset(dst, 0, size / 8 + 1);
	for (size_t i = 0; i < size; ++i)
	{
		if (src[i] > 0) { put_bit(dst, i); }
	}
}

/* ---- a2: binary_align_weights, src-lib/convolutional_layer.cpp:1339-1411 ---------------- */
/*
 * weights: [n][c*size*size] fp32 (BN already folded).  Outputs:
 *   align_bit_weights: n*new_lda/8 + 1 bytes.  Row f starts at bit f*new_lda; bits >= K are 0
 *                      (1 after inversion).
 *   mean_arr[n]:       |binary_weights[f*K]| (src-lib/convolutional_layer.cpp:131-140)
 * K order: c % 32 == 0 -> bit (cb*size*size + tap)*32 + (c - 32*cb)   (:1364-1391)
 *          otherwise   -> plain  c*size*size + tap                    (:1356-1362)
 * invert != 0 reproduces the GPU-build layout: every byte complemented when c % 32 == 0
 * (:1395-1401); the bit path is never inverted (:1406-1411).
 */
ORACLE_API void oracle_binary_align_weights(const float * weights, int n, int c, int size, int invert,
		uint8_t * align_bit_weights, float * mean_arr)
{
	const int taps = size * size;
	const int k = taps * c;
	const size_t new_lda = (size_t)oracle_new_lda(k);
	const size_t total_bits = new_lda * (size_t)n;
	float * binary = (float *)malloc(sizeof(float) * (size_t)n * k);
	oracle_binarize_weights(weights, n, k, binary);

	memset(align_bit_weights, 0, total_bits / 8 + 1);
	for (int f = 0; f < n; ++f)
	{
		for (int ch = 0; ch < c; ++ch)
		{
			for (int t = 0; t < taps; ++t)
			{
				const float v = binary[(size_t)f * k + (size_t)ch * taps + t];
				size_t bit;
				if (c % 32 == 0)
				{
					const int cb = ch / 32;
					bit = (size_t)f * new_lda + (size_t)cb * 32 * taps + (size_t)t * 32 + (ch - 32 * cb);
				}
				else
				{
					bit = (size_t)f * new_lda + (size_t)ch * taps + t;
				}
				if (v > 0) { put_bit(align_bit_weights, bit); }
			}
		}
		mean_arr[f] = fabsf(binary[(size_t)f * k]);
	}
	if (invert && c % 32 == 0)
	{
		for (size_t i = 0; i < total_bits / 8; ++i) { align_bit_weights[i] = (uint8_t)~align_bit_weights[i]; }
	}
	free(binary);
}

/* ---- a4: repack_input + float_to_bit, src-lib/gemm.cpp:2202-2220 and :1510 -------------- */
/* in [c][h*w] fp32 -> out [c/32][h*w] uint32, bit (ch%32) = in > 0.  c % 32 == 0. */
ORACLE_API void oracle_repack_input_bin(const float * in, int c, int h, int w, uint32_t * out)
{
	const size_t hw = (size_t)h * w;
	for (int cb = 0; cb < c / 32; ++cb)
	{
		for (size_t i = 0; i < hw; ++i)
		{
			uint32_t word = 0;
			for (int b = 0; b < 32; ++b)
			{
				if (in[((size_t)cb * 32 + b) * hw + i] > 0) { word |= (1u << b); }
			}
			out[(size_t)cb * hw + i] = word;
		}
	}
}

/* ---- a5: im2col over packed words, src-lib/im2col.cpp:8-49 (called at
 *      src-lib/convolutional_layer.cpp:1509 with the words reinterpreted as float) ---------- */
/* words [channels][h][w] -> col [channels*ks*ks][out_h*out_w]; out-of-image taps are word 0. */
ORACLE_API void oracle_im2col_words(const uint32_t * words, int channels, int h, int w, int ks, int stride, int pad,
		uint32_t * col)
{
	const int oh = oracle_out_dim(h, ks, stride, pad);
	const int ow = oracle_out_dim(w, ks, stride, pad);
	const int rows = channels * ks * ks;
	for (int r = 0; r < rows; ++r)
	{
		const int kx = r % ks;
		const int ky = (r / ks) % ks;
		const int ch = r / ks / ks;
		for (int y = 0; y < oh; ++y)
		{
			for (int x = 0; x < ow; ++x)
			{
				const int iy = ky + y * stride - pad;
				const int ix = kx + x * stride - pad;
				uint32_t v = 0;
				if (iy >= 0 && ix >= 0 && iy < h && ix < w) { v = words[((size_t)ch * h + iy) * w + ix]; }
				col[((size_t)r * oh + y) * ow + x] = v;
			}
		}
	}
}

/* ---- a6: transpose_uint32, src-lib/gemm.cpp:2222-2239 ----------------------------------- */
/* dst[j*dst_align/32 + i] = src[i*src_align + j]; words i >= src_h of a dst row are untouched. */
ORACLE_API void oracle_transpose_uint32(const uint32_t * src, uint32_t * dst, int src_h, int src_w, int src_align, int dst_align)
{
	for (int i = 0; i < src_h; ++i)
	{
		for (int j = 0; j < src_w; ++j)
		{
			dst[(size_t)j * dst_align / 32 + i] = src[(size_t)i * src_align + j];
		}
	}
}

/* ---- a7: im2col_cpu_custom_bin, src-lib/gemm.cpp:1339-1460 ------------------------------ */
/*
 * in [c][h][w] fp32 -> bit matrix [K][bit_align], bit (k*bit_align + p) = tap value > 0,
 * k = ch*ks*ks + ky*ks + kx, p = y*out_w + x; out-of-image taps are 0.  The reference only
 * implements the 3x3-like same-size stride-1 pad-1 case (:1351) and prints a message
 * otherwise (:1454); this generic form equals it there and is the definition elsewhere.
 * col must hold K*bit_align/8 bytes; all are written.
 */
ORACLE_API void oracle_im2col_bin(const float * in, int c, int h, int w, int ks, int stride, int pad, int bit_align,
		uint8_t * col)
{
	const int oh = oracle_out_dim(h, ks, stride, pad);
	const int ow = oracle_out_dim(w, ks, stride, pad);
	const int rows = c * ks * ks;
	memset(col, 0, (size_t)rows * bit_align / 8);
	for (int r = 0; r < rows; ++r)
	{
		const int kx = r % ks;
		const int ky = (r / ks) % ks;
		const int ch = r / ks / ks;
		for (int y = 0; y < oh; ++y)
		{
			for (int x = 0; x < ow; ++x)
			{
				const int iy = ky + y * stride - pad;
				const int ix = kx + x * stride - pad;
				if (iy >= 0 && ix >= 0 && iy < h && ix < w && in[((size_t)ch * h + iy) * w + ix] > 0)
				{
					put_bit(col, (size_t)r * bit_align + (size_t)y * ow + x);
				}
			}
		}
	}
}

/* ---- a8: transpose_bin, src-lib/gemm.cpp:216-245 (32x32 bit blocks, :120-175) ----------- */
/*
 * A: n rows of lda bits; B: m rows of ldb bits; B bit (j, i) = A bit (i, j) for i < n, j < m.
 * The reference works on whole 32x32 blocks, so it also writes rows m..ceil32(m) and columns
 * n..ceil32(n) of B from whatever lies beyond A's logical edge; callers keep those zero
 * (src-lib/convolutional_layer.cpp:1473 clears the workspace).  B is expected pre-zeroed
 * (src-lib/convolutional_layer.cpp:152).
 */
ORACLE_API void oracle_transpose_bin(const uint8_t * A, uint8_t * B, int n, int m, int lda, int ldb)
{
	for (int i = 0; i < n; ++i)
	{
		for (int j = 0; j < m; ++j)
		{
			if (read_bit(A, (size_t)i * lda + j)) { put_bit(B, (size_t)j * ldb + i); }
		}
	}
}

/* ---- a4..a8 combined: the packed, transposed B operand of one image -------------------- */
/*
 * t_bit_input [N][new_ldb/8] bytes as left by src-lib/convolutional_layer.cpp:1475-1545:
 * word path (c % 32 == 0): repack -> bits -> im2col on words -> transpose_uint32;
 * bit path: im2col_bin -> transpose_bin.  Padding bits (k >= K) are 0.
 */
ORACLE_API void oracle_pack_input(const float * in, int c, int h, int w, int ks, int stride, int pad, uint8_t * t_bit_input)
{
	const int oh = oracle_out_dim(h, ks, stride, pad);
	const int ow = oracle_out_dim(w, ks, stride, pad);
	const int n = oh * ow;
	const int k = ks * ks * c;
	const int new_ldb = oracle_new_lda(k);
	memset(t_bit_input, 0, (size_t)n * new_ldb / 8);
	if (c % 32 == 0)
	{
		const int new_c = c / 32;
		const int new_k = ks * ks * new_c;
		uint32_t * packed = (uint32_t *)calloc((size_t)new_c * h * w + 1, sizeof(uint32_t));
		uint32_t * col = (uint32_t *)calloc((size_t)new_k * n + 1, sizeof(uint32_t));
		oracle_repack_input_bin(in, c, h, w, packed);
		oracle_im2col_words(packed, new_c, h, w, ks, stride, pad, col);
		oracle_transpose_uint32(col, (uint32_t *)t_bit_input, new_k, n, n, new_ldb);
		free(col);
		free(packed);
	}
	else
	{
		const int bit_align = oracle_bit_align(n);
		uint8_t * col = (uint8_t *)calloc((size_t)k * bit_align / 8 + 8, 1);
		oracle_im2col_bin(in, c, h, w, ks, stride, pad, bit_align, col);
		oracle_transpose_bin(col, t_bit_input, k, n, bit_align, new_ldb);
		free(col);
	}
}

/* ---- a9: gemm_nn_custom_bin_mean_transposed, src-lib/gemm.cpp:907-1019 ------------------ */
/*
 * A: M rows of lda bits, B: N rows of ldb bits, both zero padded beyond K.
 * count = popcount(xnor(A_i, B_j)) over ceil256(K) bits, minus f1 = padding bits (:966);
 * i.e. the number of agreeing bits among the first K.  counts[i*N + j] receives it.
 */
ORACLE_API void oracle_gemm_counts(int M, int N, int K, const uint8_t * A, int lda, const uint8_t * B, int ldb, int32_t * counts)
{
	const int bit_step = 256;
	const int f1 = (K % bit_step == 0) ? 0 : (bit_step - (K % bit_step));
	const int kbits = K + f1;
	#pragma omp parallel for schedule(static)
	for (int i = 0; i < M; ++i)
	{
		for (int j = 0; j < N; ++j)
		{
			int count = 0;
			for (int k = 0; k < kbits; k += 64)
			{
				uint64_t a, b;
				memcpy(&a, A + ((size_t)i * lda + k) / 8, 8);
				memcpy(&b, B + ((size_t)j * ldb + k) / 8, 8);
				count += __builtin_popcountll(~(a ^ b));
			}
			counts[(size_t)i * N + j] = count - f1;
		}
	}
}

/* C[i*ldc + j] = (2*count - K) * mean_arr[i]   (src-lib/gemm.cpp:971-974) */
ORACLE_API void oracle_gemm_bin_mean_transposed(int M, int N, int K, const uint8_t * A, int lda, const uint8_t * B, int ldb,
		float * C, int ldc, const float * mean_arr)
{
	int32_t * counts = (int32_t *)malloc(sizeof(int32_t) * (size_t)M * N);
	oracle_gemm_counts(M, N, K, A, lda, B, ldb, counts);
	for (int i = 0; i < M; ++i)
	{
		for (int j = 0; j < N; ++j)
		{
			C[(size_t)i * ldc + j] = (float)(2 * counts[(size_t)i * N + j] - K) * mean_arr[i];
		}
	}
	free(counts);
}

/* ---- a10: add_bias, src-lib/convolutional_layer.cpp:1269-1289 --------------------------- */
ORACLE_API void oracle_add_bias(float * output, const float * biases, int batch, int n, int size)
{
	for (int b = 0; b < batch; ++b)
	{
		for (int i = 0; i < n; ++i)
		{
			for (int j = 0; j < size; ++j)
			{
				volatile float v = output[((size_t)b * n + i) * size + j]; /* no fused multiply-add across the store */
				output[((size_t)b * n + i) * size + j] = v + biases[i];
			}
		}
	}
}

/* leaky: src-lib/gemm.cpp:1472-1498 -- sign bit set -> x*0.1f, else x (tail: max(x, 0.1f*x)) */
ORACLE_API void oracle_activate_leaky(float * x, size_t n)
{
	for (size_t i = 0; i < n; ++i)
	{
		const float v = x[i];
		x[i] = signbit(v) ? v * 0.1f : v;
	}
}

/* ---- a11: the xnor branch of forward_convolutional_layer, src-lib/convolutional_layer.cpp:1471-1557,
 *      applied to every image of the batch (the reference returns after image 0, :1557) ---- */
/*
 * in  [batch][c][h][w], weights [n][c*ks*ks], biases [n] -> out [batch][n][out_h*out_w].
 * Optional dumps (may be NULL): t_bit_input_all [batch][N][new_ldb/8], counts_all [batch][n][N].
 */
ORACLE_API void oracle_conv_forward(const float * in, int batch, int c, int h, int w,
		const float * weights, const float * biases, int n, int ks, int stride, int pad, int leaky,
		float * out, uint8_t * t_bit_input_all, int32_t * counts_all)
{
	const int oh = oracle_out_dim(h, ks, stride, pad);
	const int ow = oracle_out_dim(w, ks, stride, pad);
	const int N = oh * ow;
	const int K = ks * ks * c;
	const int new_lda = oracle_new_lda(K);
	uint8_t * A = (uint8_t *)calloc((size_t)n * new_lda / 8 + 1, 1);
	float * mean_arr = (float *)malloc(sizeof(float) * n);
	uint8_t * B = (uint8_t *)calloc((size_t)N * new_lda / 8 + 64, 1);
	int32_t * counts = (int32_t *)malloc(sizeof(int32_t) * (size_t)n * N);
	oracle_binary_align_weights(weights, n, c, ks, 0, A, mean_arr);
	for (int b = 0; b < batch; ++b)
	{
		float * o = out + (size_t)b * n * N;
		oracle_pack_input(in + (size_t)b * c * h * w, c, h, w, ks, stride, pad, B);
		oracle_gemm_counts(n, N, K, A, new_lda, B, new_lda, counts);
		for (int i = 0; i < n; ++i)
		{
			for (int j = 0; j < N; ++j)
			{
				o[(size_t)i * N + j] = (float)(2 * counts[(size_t)i * N + j] - K) * mean_arr[i];
			}
		}
		oracle_add_bias(o, biases, 1, n, N);
		if (leaky) { oracle_activate_leaky(o, (size_t)n * N); }
		if (t_bit_input_all) { memcpy(t_bit_input_all + (size_t)b * N * new_lda / 8, B, (size_t)N * new_lda / 8); }
		if (counts_all) { memcpy(counts_all + (size_t)b * n * N, counts, sizeof(int32_t) * (size_t)n * N); }
	}
	free(counts);
	free(B);
	free(mean_arr);
	free(A);
}
