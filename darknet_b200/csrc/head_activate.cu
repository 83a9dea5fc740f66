// Activation steps of the [yolo] and [region] heads that close the xnor networks, one kernel each.
//
// forward_yolo_layer_gpu (src-lib/yolo_layer.cpp:1439-1489) applies the logistic function to the x, y entries and
// to the objectness + class entries of every anchor (two activate_array_ongpu launches per anchor and image) and
// leaves w, h raw.  The tensor is [batch][anchors][4 + 1 + classes][h*w]; one pass reads and writes it once.
// logistic(x) = 1 / (1 + expf(-x)), the form of src-lib/activation_kernels.cu (logistic_activate_kernel).
#include "xnor_common.cuh"

namespace xnor
{

__global__ void __launch_bounds__(256)
yolo_activate_kernel(const float * __restrict__ in, float * __restrict__ out, size_t total, int entries, int hw)
{
	for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256)
	{
		const int e = (int)((i / hw) % entries);
		float v = in[i];
		if (e != 2 && e != 3) { v = 1.0f / (1.0f + expf(-v)); }
		out[i] = v;
	}
}

// [region] head (src-lib/region_layer.cpp:494-537): per image, anchor and cell the logistic function on x, y and the
// objectness entry, w and h raw, and -- with softmax=1 -- a softmax over the class entries (max subtracted, temperature
// 1: softmax_cpu in src-lib/blas.cpp).  The tensor is [batch][anchors][coords + 1 + classes][h*w]; a thread owns one
// (image, anchor, cell), so every access of a warp is 32 consecutive cells of one entry plane.  The class scores
// are read twice (running maximum and sum in one pass, normalised values in the second, from L1/L2).
__global__ void __launch_bounds__(256)
region_activate_kernel(const float * __restrict__ in, float * __restrict__ out, size_t cells, int coords, int classes, int softmax, int hw)
{
	const int entries = coords + 1 + classes;
	for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < cells; i += (size_t)gridDim.x * 256)
	{
		const size_t group = i / hw;                          // image * anchors + anchor
		const size_t base = group * entries * hw + (i - group * hw);
		for (int e = 0; e <= coords; ++e)
		{
			float v = in[base + (size_t)e * hw];
			if (e < 2 || e == coords) { v = 1.0f / (1.0f + expf(-v)); }
			out[base + (size_t)e * hw] = v;
		}
		const float * cls = in + base + (size_t)(coords + 1) * hw;
		float * dst = out + base + (size_t)(coords + 1) * hw;
		if (!softmax)
		{
			for (int c = 0; c < classes; ++c) { dst[(size_t)c * hw] = cls[(size_t)c * hw]; }
			continue;
		}
		float largest = -INFINITY;
		for (int c = 0; c < classes; ++c) { largest = fmaxf(largest, cls[(size_t)c * hw]); }
		float sum = 0.0f;
		for (int c = 0; c < classes; ++c) { sum += expf(cls[(size_t)c * hw] - largest); }
		for (int c = 0; c < classes; ++c) { dst[(size_t)c * hw] = expf(cls[(size_t)c * hw] - largest) / sum; }
	}
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_region_activate(const float * input, float * output, int batch, int anchors, int coords, int classes,
		int softmax, int hw, void * stream)
{
	if (input == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	if (batch <= 0 || anchors <= 0 || coords < 2 || classes < 0 || hw <= 0 || input == output) { return XNOR_B200_ERR_INVALID; }
	const size_t cells = (size_t)batch * anchors * hw;
	const int grid = (int)min((cells + 255) / 256, (size_t)sm_count() * 8);
	region_activate_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(input, output, cells, coords, classes, softmax, hw);
	return check_launch();
}

extern "C" int xnor_b200_yolo_activate(const float * input, float * output, int batch, int anchors, int classes, int hw, void * stream)
{
	if (input == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	if (batch <= 0 || anchors <= 0 || classes < 0 || hw <= 0) { return XNOR_B200_ERR_INVALID; }
	const int entries = 4 + 1 + classes;
	const size_t total = (size_t)batch * anchors * entries * hw;
	const int grid = (int)min((total + 255) / 256, (size_t)sm_count() * 8);
	yolo_activate_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(input, output, total, entries, hw);
	return check_launch();
}
