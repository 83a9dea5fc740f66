// Activation step of the [yolo] head that closes the xnor networks, as one kernel.
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

}  // namespace xnor

using namespace xnor;

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
