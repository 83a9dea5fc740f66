// Load-time weight preparation for xnor conv layers: per-filter mean |w|, sign bits, packing.
//
// Replaces binarize_weights (src-lib/convolutional_layer.cpp:196-213), fast_binarize_weights_gpu
// (src-lib/convolutional_kernels.cu:116-132) and the host triple loop + float_to_bit of
// binary_align_weights (src-lib/convolutional_layer.cpp:1339-1411).  One CTA per filter.
//
// The mean is the reference CPU value bit for bit: |w| is accumulated in index order in fp32 by a
// single thread (coalesced chunk loads into shared memory feed it), then divided by the row length.
// That costs a few tens of microseconds per filter and runs once per network load; every other
// kernel in the path consumes mean_arr, so an order-dependent reduction here would leak rounding
// differences into every layer output.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int WP_THREADS = 256;
constexpr int WP_CHUNK = 2048;  // floats staged per step (8 KB)

// weights [n][K] fp32.  Outputs (each optional): binary [n][K] = +-mean, mean_arr [n],
// bits [n][lda_words] packed sign words.
//   word_path: bit (cb*taps + t)*32 + (ch - 32*cb)  <- weight (ch, t)      (K = c*taps, c%32==0)
//   else:      bit  ch*taps + t                      <- weight (ch, t)
// Padding bits are 0 (1 when invert).
__global__ void __launch_bounds__(WP_THREADS)
weights_pack_kernel(const float * __restrict__ weights, int K, int taps, int lda_words, int word_path, int invert,
		float * __restrict__ binary, float * __restrict__ mean_arr, uint32_t * __restrict__ bits)
{
	__shared__ float chunk[WP_CHUNK];
	__shared__ float s_mean;
	const int f = blockIdx.x;
	const float * row = weights + (size_t)f * K;

	if (binary != nullptr || mean_arr != nullptr)
	{
		float sum = 0.0f;
		for (int base = 0; base < K; base += WP_CHUNK)
		{
			const int len = min(WP_CHUNK, K - base);
			for (int i = threadIdx.x; i < len; i += WP_THREADS) { chunk[i] = fabsf(row[base + i]); }
			__syncthreads();
			if (threadIdx.x == 0)
			{
				for (int i = 0; i < len; ++i) { sum = __fadd_rn(sum, chunk[i]); }
			}
			__syncthreads();
		}
		if (threadIdx.x == 0)
		{
			const float m = __fdiv_rn(sum, (float)K);
			s_mean = m;
			if (mean_arr != nullptr) { mean_arr[f] = fabsf(m); }
		}
		__syncthreads();
		if (binary != nullptr)
		{
			const float m = s_mean;
			for (int i = threadIdx.x; i < K; i += WP_THREADS) { binary[(size_t)f * K + i] = (row[i] > 0) ? m : -m; }
		}
	}

	if (bits != nullptr)
	{
		uint32_t * out = bits + (size_t)f * lda_words;
		for (int wi = threadIdx.x; wi < lda_words; wi += WP_THREADS)
		{
			uint32_t word = 0;
			if (word_path)
			{
				const int cb = wi / taps;
				const int t = wi - cb * taps;
				if ((size_t)cb * 32 * taps < (size_t)K)
				{
					#pragma unroll 8
					for (int b = 0; b < 32; ++b)
					{
						const float v = row[(size_t)(cb * 32 + b) * taps + t];
						word |= (v > 0 ? 1u : 0u) << b;
					}
				}
			}
			else
			{
				const int k0 = wi * 32;
				for (int b = 0; b < 32 && k0 + b < K; ++b)
				{
					word |= (row[k0 + b] > 0 ? 1u : 0u) << b;
				}
			}
			out[wi] = invert ? ~word : word;
		}
	}
}

// Bit k' = t*C + c of a tap-major row is bit c*taps + t of the reference-order row ([c][tap], c % 32 != 0 layers).
__global__ void tap_major_weights_kernel(const uint32_t * __restrict__ in, uint32_t * __restrict__ out, int n, int C, int taps, int lda_words)
{
	const int idx = blockIdx.x * blockDim.x + threadIdx.x;
	if (idx >= n * lda_words) { return; }
	const int f = idx / lda_words;
	const int w = idx - f * lda_words;
	const uint32_t * row = in + (size_t)f * lda_words;
	uint32_t v = 0;
	for (int b = 0; b < 32; ++b)
	{
		const int k = w * 32 + b;
		if (k >= C * taps) { break; }
		const int t = k / C;
		const int c = k - t * C;
		const int src = c * taps + t;
		v |= ((row[src >> 5] >> (src & 31)) & 1u) << b;
	}
	out[idx] = v;
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_tap_major_weights(const xnor_b200_conv_desc * desc, const uint8_t * align_bit_weights, uint8_t * tap_major, void * stream)
{
	if (desc == nullptr || align_bit_weights == nullptr || tap_major == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (desc->c % 32 == 0) { return XNOR_B200_ERR_INVALID; }          // the c % 32 == 0 layout is tap-major inside each 32-channel block already
	if ((((uintptr_t)align_bit_weights | (uintptr_t)tap_major) & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	const int taps = desc->size * desc->size;
	const int lda_words = aligned_lda(taps * desc->c) / 32;
	const int total = desc->n * lda_words;
	tap_major_weights_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const uint32_t *)align_bit_weights, (uint32_t *)tap_major,
			desc->n, desc->c, taps, lda_words);
	return check_launch();
}

extern "C" int xnor_b200_binarize_weights(const float * weights, int n, int size, float * binary, float * mean_arr, void * stream)
{
	if (weights == nullptr || (binary == nullptr && mean_arr == nullptr)) { return XNOR_B200_ERR_NULL; }
	if (n <= 0 || size <= 0) { return XNOR_B200_ERR_INVALID; }
	weights_pack_kernel<<<n, WP_THREADS, 0, (cudaStream_t)stream>>>(weights, size, 1, 0, 0, 0, binary, mean_arr, nullptr);
	return check_launch();
}

extern "C" int xnor_b200_binary_align_weights(const xnor_b200_conv_desc * desc, const float * weights,
		uint8_t * align_bit_weights, float * mean_arr, int invert, void * stream)
{
	if (desc == nullptr || weights == nullptr || align_bit_weights == nullptr || mean_arr == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (((uintptr_t)align_bit_weights & 3u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	const int taps = desc->size * desc->size;
	const int K = taps * desc->c;
	const int lda_words = aligned_lda(K) / 32;
	const int word_path = (desc->c % 32 == 0) ? 1 : 0;
	// The reference complements the packed weights only on the c%32==0 branch
	// (src-lib/convolutional_layer.cpp:1395-1401 vs :1406-1411).
	const int inv = (invert && word_path) ? 1 : 0;
	weights_pack_kernel<<<desc->n, WP_THREADS, 0, (cudaStream_t)stream>>>(weights, K, taps, lda_words, word_path, inv,
			nullptr, mean_arr, (uint32_t *)align_bit_weights);
	return check_launch();
}
