// Test and benchmark infrastructure, not product code.
//
// Drives the reference's OWN GPU xnor kernels (src-lib/im2col_kernels.cu, compiled unmodified for sm_100a from the mounted
// tree by `make refgpu`) exactly as forward_convolutional_layer_gpu does for a c % 32 == 0 layer
// (src-lib/convolutional_kernels.cu:220-231): repack_input_gpu_bin -> im2col_ongpu -> transpose_uint32_gpu ->
// gemm_nn_custom_bin_mean_transposed_gpu (its wmma b1 tensor kernel).  This is the "kernel to beat": bench.py times it on
// BASELINE configuration 1 beside the library's own kernels.  The few host helpers those launchers call (stream, grid
// size, error check: src-lib/dark_cuda.cpp) are supplied here.
#include "darknet_internal.hpp"
#include "im2col.hpp"

static cudaStream_t g_stream = nullptr;
static int g_error = 0;

cudaStream_t get_cuda_stream() { return g_stream; }

int get_number_of_blocks(int array_size, int block_size)
{
	return array_size / block_size + ((array_size % block_size > 0) ? 1 : 0);       // src-lib/dark_cuda.cpp:682-687
}

void check_cuda_error_extended(cudaError_t status, const char * const, const char * const, const int)
{
	if (status != cudaSuccess) { g_error = (int)status; }
}

extern "C"
{

// One image through the reference chain.  Buffers (device): input [c][h][w] fp32; align_ws >= (c/32)*h*w words; workspace
// >= (c/32)*size*size*out_h*out_w words; transposed = out_h*out_w rows of new_ldb bits, ZERO-FILLED by the caller (the
// reference leaves the row padding unwritten); weights = align_bit_weights in the reference's GPU layout (complemented, see
// src-lib/convolutional_layer.cpp:1395-1401); out [n][out_h*out_w].  gemm_only != 0 skips the three input kernels.
// Requires c % 32 == 0, n >= 8, out_h*out_w >= 16 (the tensor kernel shifts its last tiles back, src-lib/im2col_kernels.cu:823-824).
__attribute__((visibility("default"))) int refgpu_xnor_chain(int c, int h, int w, int n, int size, int stride, int pad,
		float * input, float * align_ws, float * workspace, unsigned char * transposed, unsigned char * weights, float * mean_arr,
		float * biases, float * out, int leaky, int gemm_only, void * stream)
{
	if (c % 32 != 0 || n < 8) { return -1; }
	const int out_h = (h + 2 * pad - size) / stride + 1, out_w = (w + 2 * pad - size) / stride + 1;
	const int n_out = out_h * out_w, k = size * size * c;
	if (n_out < 16) { return -1; }
	const int new_ldb = k + (256 - k % 256);
	g_stream = (cudaStream_t)stream;
	g_error = 0;
	if (!gemm_only)
	{
		repack_input_gpu_bin(input, (uint32_t *)align_ws, w, h, c);
		im2col_ongpu(align_ws, c / 32, h, w, size, stride, pad, workspace);
		transpose_uint32_gpu((uint32_t *)workspace, (uint32_t *)transposed, size * size * c / 32, n_out, n_out, new_ldb);
	}
	gemm_nn_custom_bin_mean_transposed_gpu(n, n_out, k, weights, new_ldb, transposed, new_ldb, out, n_out, mean_arr, biases, leaky, nullptr, nullptr);
	return g_error;
}

}
