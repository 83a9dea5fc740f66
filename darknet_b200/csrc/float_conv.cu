// Direct fp32 convolution for the float layer that sits in FRONT of the xnor path (3 input channels -> 16 or 32
// filters at full image resolution in all three xnor networks), with bias and leaky/linear activation fused.
//
// Stands in for the float branch of forward_convolutional_layer_gpu (src-lib/convolutional_kernels.cu:373-434:
// cuDNN or im2col + cuBLAS sgemm), add_bias_gpu (src-lib/blas_kernels.cu) and activate_array_ongpu
// (src-lib/activation_kernels.cu:34 leaky) for layers with few input channels.  Such a layer is bound by writing
// its output (16 planes of the full-resolution image), not by arithmetic, so one pass that reads the image once
// and writes every output plane once, coalesced, is the whole optimisation; a GEMM formulation would only add an
// im2col buffer.  Accumulation order is (channel, ky, kx) with fused multiply-adds, bias added last.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int FC_THREADS = 256;
constexpr int FC_MAX_TAPS = 128;     // c*size*size values a thread keeps in registers
constexpr int FC_FILTERS = 16;       // filters accumulated per pass

struct FloatConvParams
{
	const float * in;
	const float * weights;   // [n][c*size*size]
	const float * biases;    // [n] or nullptr
	float * out;             // [batch][n][oh][ow]
	int batch, C, H, W, N, OH, OW;
	int ks, stride, pad;
	int leaky;
};

// CC, KS > 0: channel count and kernel size known at compile time (the 27 taps of a 3x3 RGB layer then live in
// registers); CC == 0: generic sizes, taps kept in a per-thread array.
template <int CC, int KS>
__global__ void __launch_bounds__(FC_THREADS)
float_conv_small_kernel(const FloatConvParams p)
{
	constexpr int TAPS_MAX = (CC > 0) ? CC * KS * KS : FC_MAX_TAPS;
	const int C = (CC > 0) ? CC : p.C;
	const int ks = (CC > 0) ? KS : p.ks;
	extern __shared__ float s_w[];                       // weights [n][taps] followed by biases [n]
	const int taps = C * ks * ks;
	for (int i = threadIdx.x; i < p.N * taps; i += FC_THREADS) { s_w[i] = p.weights[i]; }
	float * s_b = s_w + p.N * taps;
	for (int i = threadIdx.x; i < p.N; i += FC_THREADS) { s_b[i] = (p.biases != nullptr) ? p.biases[i] : 0.0f; }
	__syncthreads();

	const size_t plane = (size_t)p.OH * p.OW;
	const size_t total = (size_t)p.batch * plane;
	for (size_t idx = (size_t)blockIdx.x * FC_THREADS + threadIdx.x; idx < total; idx += (size_t)gridDim.x * FC_THREADS)
	{
		const int b = (int)(idx / plane);
		const int pix = (int)(idx - (size_t)b * plane);
		const int oy = pix / p.OW;
		const int ox = pix - oy * p.OW;
		const float * img = p.in + (size_t)b * C * p.H * p.W;

		float v[TAPS_MAX];
		int t = 0;
		#pragma unroll
		for (int c = 0; c < C; ++c)
		{
			#pragma unroll
			for (int ky = 0; ky < ks; ++ky)
			{
				const int iy = oy * p.stride - p.pad + ky;
				#pragma unroll
				for (int kx = 0; kx < ks; ++kx, ++t)
				{
					const int ix = ox * p.stride - p.pad + kx;
					const bool ok = (iy >= 0 && iy < p.H && ix >= 0 && ix < p.W);
					if (t < TAPS_MAX) { v[t] = ok ? __ldg(img + ((size_t)c * p.H + iy) * p.W + ix) : 0.0f; }
				}
			}
		}
		float * dst = p.out + (size_t)b * p.N * plane + pix;
		for (int f0 = 0; f0 < p.N; f0 += FC_FILTERS)
		{
			float acc[FC_FILTERS];
			#pragma unroll
			for (int f = 0; f < FC_FILTERS; ++f) { acc[f] = 0.0f; }
			#pragma unroll
			for (int k = 0; k < TAPS_MAX; ++k)
			{
				if (k < taps)
				{
					#pragma unroll
					for (int f = 0; f < FC_FILTERS; ++f)
					{
						if (f0 + f < p.N) { acc[f] = fmaf(v[k], s_w[(f0 + f) * taps + k], acc[f]); }
					}
				}
			}
			#pragma unroll
			for (int f = 0; f < FC_FILTERS; ++f)
			{
				if (f0 + f < p.N)
				{
					float r = acc[f] + s_b[f0 + f];
					if (p.leaky) { r = (r > 0.0f) ? r : r * 0.1f; }
					dst[(size_t)(f0 + f) * plane] = r;
				}
			}
		}
	}
}

// ---- 3 input channels, 3x3, stride 1, pad 1: a thread computes a 2x2 block of outputs for 8 filters ----------
// The first layer of every xnor network.  One thread loads the 4x4x3 input patch of its block once (48 values in
// registers) and reads each weight once per block as part of a 16-byte vector, so the kernel runs at FMA speed
// instead of one shared-memory load per multiply.  Three ways to finish, chosen by the caller:
//   * fp32 output at full resolution (bias, leaky/linear);
//   * the [maxpool] size 2 / stride 2 that follows the layer applied in registers, fp32 output at half resolution
//     (leaky is monotonic, so max(act(v)) == act(max(v)) value for value);
//   * only the SIGN of that pooled output, as x-packed bit planes uint32 [image][filter][H/2][ceil(W/2/32)] -- what
//     a following xnor layer needs and nothing more (max > 0 exactly when one of the four values is > 0).
// Each output value is formed exactly as in float_conv_small_kernel: fmaf over (channel, ky, kx) from zero, then
// + bias, so the three variants and that kernel agree bit for bit.
constexpr int FB_THREADS = 256;          // 8 warps: warp w = block row w of the tile, lane = block column
constexpr int FB_FILTERS = 8;            // filters per thread (blockIdx.y picks the group)

struct FloatBlockParams
{
	const float * in;        // [batch][3][H][W]
	const float * weights;   // [n][27]
	const float * biases;    // [n] or nullptr
	float * out;             // fp32 output (full or pooled) or nullptr
	uint32_t * planes;       // pooled sign planes or nullptr
	uint8_t * masks;         // pooled sign masks [image][H/2][W/2][ceil(N/8)] (bit f%8 of byte f/8) or nullptr
	int H, W, N;
	int BH, BW;              // 2x2 blocks per column / row: ceil(H/2), ceil(W/2)
	int xtiles;              // ceil(BW / 32)
	int pooled;              // 1: one value per block
	int leaky;
};

__global__ void __launch_bounds__(FB_THREADS)
float_conv3_block_kernel(const FloatBlockParams p)
{
	__shared__ __align__(16) float s_w[27 * FB_FILTERS];      // [tap][filter of this group]
	__shared__ float s_b[FB_FILTERS];
	const int f0 = blockIdx.y * FB_FILTERS;
	for (int i = threadIdx.x; i < 27 * FB_FILTERS; i += FB_THREADS)
	{
		const int k = i / FB_FILTERS;
		const int f = f0 + (i - k * FB_FILTERS);
		s_w[i] = (f < p.N) ? p.weights[(size_t)f * 27 + k] : 0.0f;
	}
	if (threadIdx.x < FB_FILTERS)
	{
		const int f = f0 + threadIdx.x;
		s_b[threadIdx.x] = (p.biases != nullptr && f < p.N) ? p.biases[f] : 0.0f;
	}
	__syncthreads();

	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	const int xt = blockIdx.x % p.xtiles;
	const int yt = blockIdx.x / p.xtiles;
	const int bx = xt * 32 + lane;
	const int by = yt * 8 + warp;
	const bool live = (bx < p.BW && by < p.BH);
	const float * img = p.in + (size_t)blockIdx.z * 3 * p.H * p.W;

	// the 4x4 patch of each channel: rows 2by-1 .. 2by+2, columns 2bx-1 .. 2bx+2
	float v[3][4][4];
	#pragma unroll
	for (int c = 0; c < 3; ++c)
	{
		#pragma unroll
		for (int r = 0; r < 4; ++r)
		{
			const int iy = 2 * by - 1 + r;
			#pragma unroll
			for (int q = 0; q < 4; ++q)
			{
				const int ix = 2 * bx - 1 + q;
				const bool ok = live && iy >= 0 && iy < p.H && ix >= 0 && ix < p.W;
				v[c][r][q] = ok ? __ldg(img + ((size_t)c * p.H + iy) * p.W + ix) : 0.0f;
			}
		}
	}
	float acc[FB_FILTERS][4];              // [filter][2*dy + dx]
	#pragma unroll
	for (int f = 0; f < FB_FILTERS; ++f)
	{
		#pragma unroll
		for (int o = 0; o < 4; ++o) { acc[f][o] = 0.0f; }
	}
	#pragma unroll
	for (int c = 0; c < 3; ++c)
	{
		#pragma unroll
		for (int ky = 0; ky < 3; ++ky)
		{
			#pragma unroll
			for (int kx = 0; kx < 3; ++kx)
			{
				const int k = (c * 3 + ky) * 3 + kx;
				const float4 wa = *reinterpret_cast<const float4 *>(s_w + k * FB_FILTERS);
				const float4 wb = *reinterpret_cast<const float4 *>(s_w + k * FB_FILTERS + 4);
				const float w[FB_FILTERS] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
				#pragma unroll
				for (int f = 0; f < FB_FILTERS; ++f)
				{
					acc[f][0] = fmaf(v[c][ky][kx], w[f], acc[f][0]);
					acc[f][1] = fmaf(v[c][ky][kx + 1], w[f], acc[f][1]);
					acc[f][2] = fmaf(v[c][ky + 1][kx], w[f], acc[f][2]);
					acc[f][3] = fmaf(v[c][ky + 1][kx + 1], w[f], acc[f][3]);
				}
			}
		}
	}

	const bool col1 = (2 * bx + 1 < p.W);
	const bool row1 = (2 * by + 1 < p.H);
	if (p.masks != nullptr && !p.pooled)
	{
		// sign of this thread's 8 filters at each of its four pixels, one byte of each pixel's channel mask; with 32
		// filters the four bytes of a pixel are the channel-packed sign word an xnor layer over 32 channels reads
		uint32_t m0 = 0, m1 = 0, m2 = 0, m3 = 0;
		#pragma unroll
		for (int f = 0; f < FB_FILTERS; ++f)
		{
			const uint32_t on = (f0 + f < p.N) ? 1u : 0u;
			m0 |= (on & (acc[f][0] + s_b[f] > 0.0f ? 1u : 0u)) << f;
			m1 |= (on & (acc[f][1] + s_b[f] > 0.0f ? 1u : 0u)) << f;
			m2 |= (on & (acc[f][2] + s_b[f] > 0.0f ? 1u : 0u)) << f;
			m3 |= (on & (acc[f][3] + s_b[f] > 0.0f ? 1u : 0u)) << f;
		}
		if (live)
		{
			uint8_t * dst = p.masks + (((size_t)blockIdx.z * p.H + 2 * by) * p.W + 2 * bx) * gridDim.y + blockIdx.y;
			dst[0] = (uint8_t)m0;
			if (col1) { dst[gridDim.y] = (uint8_t)m1; }
			if (row1)
			{
				dst[(size_t)p.W * gridDim.y] = (uint8_t)m2;
				if (col1) { dst[(size_t)(p.W + 1) * gridDim.y] = (uint8_t)m3; }
			}
		}
		return;
	}
	if (p.masks != nullptr)
	{
		// pooled sign of this thread's 8 filters as one byte of the pixel's channel mask
		uint32_t m = 0;
		#pragma unroll
		for (int f = 0; f < FB_FILTERS; ++f)
		{
			const float r0 = acc[f][0] + s_b[f], r1 = acc[f][1] + s_b[f], r2 = acc[f][2] + s_b[f], r3 = acc[f][3] + s_b[f];
			m |= ((f0 + f < p.N) && (r0 > 0.0f || r1 > 0.0f || r2 > 0.0f || r3 > 0.0f) ? 1u : 0u) << f;
		}
		if (live) { p.masks[(((size_t)blockIdx.z * p.BH + by) * p.BW + bx) * gridDim.y + blockIdx.y] = (uint8_t)m; }
		return;
	}
	#pragma unroll
	for (int f = 0; f < FB_FILTERS; ++f)
	{
		const float r0 = acc[f][0] + s_b[f], r1 = acc[f][1] + s_b[f], r2 = acc[f][2] + s_b[f], r3 = acc[f][3] + s_b[f];
		if (p.planes != nullptr)
		{
			// pooled sign: the block lies inside the image whenever it is live (H and W are even in this mode)
			const uint32_t word = __ballot_sync(0xffffffffu, live && (r0 > 0.0f || r1 > 0.0f || r2 > 0.0f || r3 > 0.0f));
			if (lane == 0 && by < p.BH && f0 + f < p.N)
			{
				p.planes[(((size_t)blockIdx.z * p.N + f0 + f) * p.BH + by) * p.xtiles + xt] = word;
			}
			continue;
		}
		if (!live || f0 + f >= p.N) { continue; }
		if (p.pooled)
		{
			float m = fmaxf(fmaxf(r0, r1), fmaxf(r2, r3));
			if (p.leaky) { m = (m > 0.0f) ? m : m * 0.1f; }
			p.out[(((size_t)blockIdx.z * p.N + f0 + f) * p.BH + by) * p.BW + bx] = m;
		}
		else
		{
			float a0 = r0, a1 = r1, a2 = r2, a3 = r3;
			if (p.leaky)
			{
				a0 = (a0 > 0.0f) ? a0 : a0 * 0.1f; a1 = (a1 > 0.0f) ? a1 : a1 * 0.1f;
				a2 = (a2 > 0.0f) ? a2 : a2 * 0.1f; a3 = (a3 > 0.0f) ? a3 : a3 * 0.1f;
			}
			float * dst = p.out + (((size_t)blockIdx.z * p.N + f0 + f) * p.H + 2 * by) * p.W + 2 * bx;
			dst[0] = a0;
			if (col1) { dst[1] = a1; }
			if (row1)
			{
				dst[p.W] = a2;
				if (col1) { dst[p.W + 1] = a3; }
			}
		}
	}
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_float_conv_small(const xnor_b200_conv_desc * desc, const float * input, const float * weights,
		const float * biases, float * output, void * stream)
{
	if (desc == nullptr || input == nullptr || weights == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	const int taps = desc->c * desc->size * desc->size;
	if (taps > FC_MAX_TAPS || desc->n > 256) { return XNOR_B200_ERR_TOO_LARGE; }
	FloatConvParams p;
	p.in = input; p.weights = weights; p.biases = biases; p.out = output;
	p.batch = desc->batch; p.C = desc->c; p.H = desc->h; p.W = desc->w; p.N = desc->n;
	p.OH = conv_out_dim(desc->h, desc->size, desc->stride, desc->pad);
	p.OW = conv_out_dim(desc->w, desc->size, desc->stride, desc->pad);
	p.ks = desc->size; p.stride = desc->stride; p.pad = desc->pad;
	p.leaky = (desc->activation == XNOR_B200_LEAKY) ? 1 : 0;
	const size_t total = (size_t)p.batch * p.OH * p.OW;
	const size_t smem = ((size_t)p.N * taps + p.N) * sizeof(float);
	const int grid = (int)min((total + FC_THREADS - 1) / FC_THREADS, (size_t)sm_count() * 8);
	if (desc->c == 3 && desc->size == 3)
	{
		rc = ensure_dynamic_smem((const void *)float_conv_small_kernel<3, 3>, smem);
		if (rc != XNOR_B200_OK) { return rc; }
		float_conv_small_kernel<3, 3><<<grid, FC_THREADS, smem, (cudaStream_t)stream>>>(p);
	}
	else
	{
		rc = ensure_dynamic_smem((const void *)float_conv_small_kernel<0, 0>, smem);
		if (rc != XNOR_B200_OK) { return rc; }
		float_conv_small_kernel<0, 0><<<grid, FC_THREADS, smem, (cudaStream_t)stream>>>(p);
	}
	return check_launch();
}

extern "C" int xnor_b200_float_conv3_io(const xnor_b200_conv_desc * desc, int pool, const float * input, const float * weights,
		const float * biases, float * output, uint32_t * output_sign_planes, uint8_t * output_sign_masks, void * stream)
{
	if (desc == nullptr || input == nullptr || weights == nullptr) { return XNOR_B200_ERR_NULL; }
	if ((output != nullptr) + (output_sign_planes != nullptr) + (output_sign_masks != nullptr) != 1) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (desc->c != 3 || desc->size != 3 || desc->stride != 1 || desc->pad != 1) { return XNOR_B200_ERR_INVALID; }
	if (pool != 0 && pool != 2) { return XNOR_B200_ERR_INVALID; }
	if (pool == 2 && (desc->h % 2 != 0 || desc->w % 2 != 0)) { return XNOR_B200_ERR_INVALID; }
	if (output_sign_planes != nullptr && pool != 2) { return XNOR_B200_ERR_INVALID; }
	FloatBlockParams p;
	p.in = input; p.weights = weights; p.biases = biases; p.out = output; p.planes = output_sign_planes; p.masks = output_sign_masks;
	p.H = desc->h; p.W = desc->w; p.N = desc->n;
	p.BH = (desc->h + 1) / 2; p.BW = (desc->w + 1) / 2;
	p.xtiles = (p.BW + 31) / 32;
	p.pooled = (pool == 2) ? 1 : 0;
	p.leaky = (desc->activation == XNOR_B200_LEAKY) ? 1 : 0;
	const long long tiles = (long long)p.xtiles * ((p.BH + 7) / 8);
	const int groups = (desc->n + FB_FILTERS - 1) / FB_FILTERS;
	if (tiles > 0x7fffffffLL || groups > 65535 || desc->batch > 65535) { return XNOR_B200_ERR_TOO_LARGE; }
	float_conv3_block_kernel<<<dim3((unsigned)tiles, (unsigned)groups, (unsigned)desc->batch), FB_THREADS, 0, (cudaStream_t)stream>>>(p);
	return check_launch();
}
