// xnor_b200_conv_forward_static: the per-layer forward for callers that must not allocate.
//
// Some hosts of this library cannot hand it a scratch buffer: a plugin slot that only receives the layer's
// input and output pointers, an inference server whose memory pool is frozen after start-up, or code running
// where cudaMalloc would synchronise the device in the middle of a latency-critical loop.  For them the packed
// activation operand lives in a fixed array inside the library image instead of in caller-provided scratch.
//
// The array is an ordinary __device__ variable, so every GPU that loads this library carries it until the
// process exits, used or not; that is why its size is kept modest.  Its name is only meaningful in device
// code: on the host the symbol is a stand-in, and its device address has to be looked up with
// cudaGetSymbolAddress, per device, with that device current.
#include "xnor_common.cuh"

#include <mutex>

namespace xnor
{

// 8 MiB covers every xnor layer of the shipped networks at batch 1 (largest: 50176 rows x 512 bits = 3.1 MiB
// in darknet53_448_xnor) and BASELINE-sized single layers up to batch 32 (676 rows x 2560 bits each).
constexpr size_t STATIC_SCRATCH_BYTES = XNOR_B200_STATIC_SCRATCH_BYTES;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static std::mutex g_static_mu;
static void * g_static_ptr[MAX_DEVICES] = {nullptr};

// Device address of g_static_scratch on the CURRENT device; resolved on first use per device.
static int static_scratch_address(void ** out)
{
	int dev = 0;
	cudaError_t e = cudaGetDevice(&dev);
	if (e != cudaSuccess) { return cuda_fail(e); }
	if (dev < 0 || dev >= MAX_DEVICES) { return XNOR_B200_ERR_INVALID; }
	std::lock_guard<std::mutex> lock(g_static_mu);
	if (g_static_ptr[dev] == nullptr)
	{
		void * p = nullptr;
		e = cudaGetSymbolAddress(&p, g_static_scratch);
		if (e != cudaSuccess) { return cuda_fail(e); }
		if (p == nullptr || (((uintptr_t)p) & 255u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
		g_static_ptr[dev] = p;
	}
	*out = g_static_ptr[dev];
	return XNOR_B200_OK;
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_conv_forward_static(const xnor_b200_conv_desc * desc, const float * input,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		float * output, const float * shortcut_in, float * shortcut_out, void * stream)
{
	if (desc == nullptr || input == nullptr || align_bit_weights == nullptr || mean_arr == nullptr || output == nullptr)
	{
		return XNOR_B200_ERR_NULL;
	}
	xnor_b200_conv_geom g;
	int rc = xnor_b200_conv_geometry(desc, &g);
	if (rc != XNOR_B200_OK) { return rc; }
	// The packed operand of the whole batch has to fit the fixed array: refuse, never truncate.
	if (g.packed_input_bytes > STATIC_SCRATCH_BYTES) { return XNOR_B200_ERR_TOO_LARGE; }
	if ((((uintptr_t)align_bit_weights) & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	if (shortcut_out != nullptr && shortcut_in == nullptr) { return XNOR_B200_ERR_NULL; }

	void * scratch = nullptr;
	rc = static_scratch_address(&scratch);
	if (rc != XNOR_B200_OK) { return rc; }

	// Nothing in the array has to start at zero: the pack kernel writes every word of every row it owns,
	// padding words included, and the GEMM reads only those rows.  What the previous call left behind in
	// the rest of the array is never read.
	cudaStream_t s = (cudaStream_t)stream;
	rc = launch_pack_input(*desc, nullptr, input, (uint32_t *)scratch, s);
	if (rc != XNOR_B200_OK) { return rc; }
	return launch_xnor_gemm(desc->n, desc->batch * g.n_out, g.n_out, g.k,
			(const uint32_t *)align_bit_weights, g.new_lda / 32, (const uint32_t *)scratch, g.new_lda / 32,
			output, g.n_out, mean_arr, biases, desc->activation == XNOR_B200_LEAKY,
			shortcut_in, shortcut_out, nullptr, s);
}
