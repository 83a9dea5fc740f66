// The adapter a Darknet maintainer adds to src-lib/ to run every [convolutional] xnor=1 layer through libxnor_b200.so.
//
// Seam: Darknet's per-layer function pointer forward_gpu (src-lib/darknet_layers.hpp:30), assigned in
// make_convolutional_layer (src-lib/convolutional_layer.cpp:916) and already re-assigned by Darknet itself at load time
// for fused shortcuts (src-lib/darknet_network.cpp:1809-1810).  Call xnor_b200_attach() once, right after
// load_network_custom() (src-lib/weights.cpp:665-691) has run fuse_conv_batchnorm and calculate_binary_weights; nothing
// else of Darknet changes.  Build with -DDARKNET_GPU (as Darknet's own CUDA build does), add include/ of this repository
// to the include path and link libxnor_b200.so.
//
// This file is compiled by tests/test_boundary_compile.py against the reference headers wherever the reference tree is
// mounted, so the field names and signatures used here are checked against the real Darknet::Layer / NetworkState.
#include "darknet_internal.hpp"
#include "xnor_b200.h"

#include <vector>

namespace
{
	struct XnorSlot { uint8_t * bits; float * mean; void * scratch; size_t scratch_bytes; };
	std::vector<XnorSlot> slots;                         // indexed by layer index

	xnor_b200_conv_desc describe(const Darknet::Layer & l)
	{
		xnor_b200_conv_desc d;
		d.batch = l.batch; d.c = l.c; d.h = l.h; d.w = l.w; d.n = l.n;
		d.size = l.size; d.stride = l.stride; d.pad = l.pad;
		d.activation = (l.activation == LEAKY) ? XNOR_B200_LEAKY : XNOR_B200_LINEAR;
		return d;
	}

	void forward_xnor_b200(Darknet::Layer & l, Darknet::NetworkState state)
	{
		const XnorSlot & s = slots[l.index];
		const xnor_b200_conv_desc d = describe(l);
		const int rc = xnor_b200_conv_forward(&d, state.input, s.bits, s.mean, l.biases_gpu, l.output_gpu,
		                                      l.bin_conv_shortcut_in_gpu, l.bin_conv_shortcut_out_gpu,
		                                      s.scratch, s.scratch_bytes, get_cuda_stream());
		if (rc != XNOR_B200_OK) { darknet_fatal_error(DARKNET_LOC, "xnor_b200_conv_forward: %s", xnor_b200_strerror(rc)); }
		// activations other than linear/leaky stay where Darknet applies them (src-lib/convolutional_kernels.cu:253-259)
	}
}

void xnor_b200_attach(Darknet::Network & net)
{
	slots.assign(net.n, XnorSlot());
	for (int j = 0; j < net.n; ++j)
	{
		Darknet::Layer & l = net.layers[j];
		if (l.type != Darknet::ELayerType::CONVOLUTIONAL || !l.xnor || l.stride_x != l.stride_y) { continue; }
		if (l.activation != LEAKY && l.activation != LINEAR) { continue; }   // keep Darknet's path for exotic activations
		const xnor_b200_conv_desc d = describe(l);
		xnor_b200_conv_geom g;
		if (xnor_b200_conv_geometry(&d, &g) != XNOR_B200_OK) { continue; }
		XnorSlot & s = slots[j];
		CHECK_CUDA(cudaMalloc((void **)&s.bits, g.weights_bytes));
		CHECK_CUDA(cudaMalloc((void **)&s.mean, sizeof(float) * l.n));
		s.scratch_bytes = xnor_b200_scratch_bytes(&d);
		CHECK_CUDA(cudaMalloc(&s.scratch, s.scratch_bytes));
		// l.weights_gpu holds the BN-folded fp32 weights (push_convolutional_layer in fuse_conv_batchnorm)
		const int rc = xnor_b200_binary_align_weights(&d, l.weights_gpu, s.bits, s.mean, /*invert=*/0, get_cuda_stream());
		if (rc != XNOR_B200_OK) { darknet_fatal_error(DARKNET_LOC, "xnor_b200_binary_align_weights: %s", xnor_b200_strerror(rc)); }
		// the two bit_align*K*4-byte buffers binary_align_weights allocated per layer are never touched again
		if (l.align_workspace_gpu) { cuda_free(l.align_workspace_gpu); l.align_workspace_gpu = nullptr; }
		if (l.transposed_align_workspace_gpu) { cuda_free(l.transposed_align_workspace_gpu); l.transposed_align_workspace_gpu = nullptr; }
		l.forward_gpu = forward_xnor_b200;
	}
	CHECK_CUDA(cudaStreamSynchronize(get_cuda_stream()));
}
