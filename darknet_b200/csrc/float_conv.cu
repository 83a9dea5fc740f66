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
