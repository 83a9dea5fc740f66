// Test infrastructure, not product code.
//
// Thin extern "C" driver around the reference's OWN xnor CPU sources (gemm.cpp, im2col.cpp,
// activations.cpp, convolutional_layer.cpp), which the Makefile in this directory compiles
// unmodified from the mounted reference tree.  Nothing from those sources is copied here:
// this file only (a) supplies link-time definitions for reference symbols that live in
// translation units we do not build (all unreachable from the xnor forward path and
// therefore abort()), and (b) exports flat C wrappers so the Python tests can call the
// reference functions and compare them with the C restatement in xnor_oracle.c and with
// the CUDA path.
//
// Built only where the reference tree is available; the resulting liboracle_ref.so lands
// in oracle/_ref/ and is never linked or loaded by the product library.

#include "darknet_internal.hpp"
#include "gemm.hpp"
#include "im2col.hpp"
#include "convolutional_layer.hpp"
#include "activations.hpp"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

// ---------------------------------------------------------------------------------------
// (a) link-time stand-ins for reference symbols outside the compiled subset
// ---------------------------------------------------------------------------------------

#define ORACLE_UNREACHABLE(name) do { std::fprintf(stderr, "oracle/_ref: unreachable reference symbol called: %s\n", name); std::abort(); } while (0)

Darknet::CfgAndState::CfgAndState()
{
	// CPU semantics by default (src-lib/convolutional_layer.cpp:1395 tests gpu_index >= 0).
	gpu_index = -1;
	output = &std::cout;
}
Darknet::CfgAndState::~CfgAndState() {}
Darknet::CfgAndState & Darknet::CfgAndState::get()
{
	static CfgAndState instance;
	return instance;
}
Darknet::ArgsAndParms::~ArgsAndParms() {}

void darknet_fatal_error(const char * const filename, const char * const funcname, const int line, const char * const msg, ...)
{
	std::fprintf(stderr, "oracle/_ref: darknet_fatal_error at %s:%s:%d: %s\n", filename, funcname, line, msg);
	std::abort();
}

void * xcalloc_location(const size_t nmemb, const size_t size, const char * const, const char * const, const int)
{
	void * p = std::calloc(nmemb ? nmemb : 1, size ? size : 1);
	if (!p) { std::abort(); }
	return p;
}
void * xrealloc_location(void * ptr, const size_t size, const char * const, const char * const, const int)
{
	void * p = std::realloc(ptr, size ? size : 1);
	if (!p) { std::abort(); }
	return p;
}

// The layer constructor fills weights with random values; the tests overwrite them.
void rand_uniform_many(float * x, const size_t n, float, float, const float) { std::memset(x, 0, n * sizeof(float)); }

// src-lib/convolutional_layer.cpp:1444 zeroes the output through this BLAS helper.
void fill_cpu(int N, float ALPHA, float * X, int INCX) { for (int i = 0; i < N; ++i) { X[i * INCX] = ALPHA; } }

void axpy_cpu(int, float, float *, int, float *, int) { ORACLE_UNREACHABLE("axpy_cpu"); }
void scal_cpu(int, float, float *, int) { ORACLE_UNREACHABLE("scal_cpu"); }
float sum_array(float *, int) { ORACLE_UNREACHABLE("sum_array"); }
void forward_batchnorm_layer(Darknet::Layer &, Darknet::NetworkState) { ORACLE_UNREACHABLE("forward_batchnorm_layer"); }
void backward_batchnorm_layer(Darknet::Layer &, Darknet::NetworkState) { ORACLE_UNREACHABLE("backward_batchnorm_layer"); }
void col2im_cpu_ext(const float *, const int, const int, const int, const int, const int, const int, const int, const int, const int, const int, const int, float *) { ORACLE_UNREACHABLE("col2im_cpu_ext"); }
Darknet::Box float_to_box_stride(const float *, const int) { ORACLE_UNREACHABLE("float_to_box_stride"); }

namespace Darknet
{
	Image collapse_image_layers(const Image &, int) { ORACLE_UNREACHABLE("collapse_image_layers"); }
	Image copy_image(const Image &) { ORACLE_UNREACHABLE("copy_image"); }
	Image float_to_image(int, int, int, float *) { ORACLE_UNREACHABLE("float_to_image"); }
	void free_image(Image &) { ORACLE_UNREACHABLE("free_image"); }
	void normalize_image(Image &) { ORACLE_UNREACHABLE("normalize_image"); }
	void rgbgr_image(Image &) { ORACLE_UNREACHABLE("rgbgr_image"); }
	void scale_image(Image &, float) { ORACLE_UNREACHABLE("scale_image"); }
	void show_image(const Image &, const char *) { ORACLE_UNREACHABLE("show_image"); }
	void show_images(Image *, int, const char *) { ORACLE_UNREACHABLE("show_images"); }
}

// ---------------------------------------------------------------------------------------
// (b) flat C exports
// ---------------------------------------------------------------------------------------

// transpose_bin is compiled only in CPU builds of the reference (src-lib/gemm.cpp:94-247)
// and has no declaration visible here.
void transpose_bin(uint32_t * A, uint32_t * B, const int n, const int m, const int lda, const int ldb, const int block_size);

struct RefLayer
{
	Darknet::Layer l;
	float * workspace;
};

extern "C"
{

void ref_set_gpu_index(int idx) { Darknet::CfgAndState::get().gpu_index = idx; }

void ref_set_num_threads(int n)
{
#ifdef DARKNET_OPENMP
	omp_set_num_threads(n);
#else
	(void)n;
#endif
}

int ref_max_threads()
{
#ifdef DARKNET_OPENMP
	return omp_get_max_threads();
#else
	return 1;
#endif
}

// ---- stage-level wrappers: one per reference function on the path ----

void ref_binarize_weights(float * weights, int n, int size, float * binary) { binarize_weights(weights, n, size, binary); }
void ref_float_to_bit(float * src, unsigned char * dst, size_t size) { float_to_bit(src, dst, size); }
void ref_repack_input(float * input, float * re_packed, int w, int h, int c) { repack_input(input, re_packed, w, h, c); }
void ref_im2col_cpu_custom(float * im, int channels, int height, int width, int ksize, int stride, int pad, float * col) { im2col_cpu_custom(im, channels, height, width, ksize, stride, pad, col); }
void ref_transpose_uint32(uint32_t * src, uint32_t * dst, int src_h, int src_w, int src_align, int dst_align) { transpose_uint32(src, dst, src_h, src_w, src_align, dst_align); }
void ref_im2col_cpu_custom_bin(float * im, int channels, int height, int width, int ksize, int stride, int pad, float * col, int bit_align) { im2col_cpu_custom_bin(im, channels, height, width, ksize, stride, pad, col, bit_align); }
void ref_transpose_bin(uint32_t * A, uint32_t * B, int n, int m, int lda, int ldb, int block_size) { transpose_bin(A, B, n, m, lda, ldb, block_size); }
void ref_gemm_nn_custom_bin_mean_transposed(int M, int N, int K, unsigned char * A, int lda, unsigned char * B, int ldb, float * C, int ldc, float * mean_arr)
{
	gemm_nn_custom_bin_mean_transposed(M, N, K, 1.0f, A, lda, B, ldb, C, ldc, mean_arr);
}
void ref_add_bias(float * output, float * biases, int batch, int n, int size) { add_bias(output, biases, batch, n, size); }
void ref_activate_array_cpu_custom(float * x, int n, int leaky) { activate_array_cpu_custom(x, n, leaky ? LEAKY : LINEAR); }

// ---- whole-layer wrapper: the reference's own constructor, weight packer and CPU forward ----

// Builds a batch-1 xnor conv layer with the reference constructor
// (src-lib/convolutional_layer.cpp:715), installs the caller's weights and biases and runs
// binary_align_weights (src-lib/convolutional_layer.cpp:1339).
void * ref_layer_create(int h, int w, int c, int n, int size, int stride, int pad, int leaky, const float * weights, const float * biases)
{
	RefLayer * r = new RefLayer();
	r->l = make_convolutional_layer(1, 1, h, w, c, n, 1, size, stride, stride, 1, pad, leaky ? LEAKY : LINEAR,
			0, 0, 1, 0, 0, 0, 0, nullptr, 0, 0, 0);
	std::memcpy(r->l.weights, weights, sizeof(float) * r->l.nweights);
	std::memcpy(r->l.biases, biases, sizeof(float) * n);
	binary_align_weights(&r->l);
	const size_t ws = r->l.workspace_size + 64;
	r->workspace = (float *)std::calloc(ws, 1);
	return r;
}

void ref_layer_geometry(void * handle, int * out)
{
	const Darknet::Layer & l = ((RefLayer *)handle)->l;
	out[0] = l.out_h;
	out[1] = l.out_w;
	out[2] = l.bit_align;
	out[3] = (int)l.new_lda;
	out[4] = (int)l.align_bit_weights_size;
	out[5] = l.lda_align;
	out[6] = (int)l.workspace_size;
}

const char * ref_layer_align_bit_weights(void * handle) { return ((RefLayer *)handle)->l.align_bit_weights; }
const float * ref_layer_mean_arr(void * handle) { return ((RefLayer *)handle)->l.mean_arr; }
const float * ref_layer_binary_weights(void * handle) { return ((RefLayer *)handle)->l.binary_weights; }
const char * ref_layer_t_bit_input(void * handle) { return ((RefLayer *)handle)->l.t_bit_input; }
const uint32_t * ref_layer_bin_re_packed_input(void * handle) { return ((RefLayer *)handle)->l.bin_re_packed_input; }

// Runs forward_convolutional_layer (src-lib/convolutional_layer.cpp:1437) on one image and
// copies l.output (n * out_h * out_w floats) to `output`.
void ref_layer_forward(void * handle, const float * input, float * output)
{
	RefLayer * r = (RefLayer *)handle;
	Darknet::NetworkState state;
	std::memset((void *)&state, 0, sizeof(state));
	state.input = const_cast<float *>(input);
	state.workspace = r->workspace;
	state.train = 0;
	forward_convolutional_layer(r->l, state);
	std::memcpy(output, r->l.output, sizeof(float) * r->l.outputs);
}

void ref_layer_destroy(void * handle)
{
	RefLayer * r = (RefLayer *)handle;
	std::free(r->workspace);
	// Layer-owned host buffers are released with the process; the reference's free_layer
	// lives in a translation unit outside the compiled subset.
	delete r;
}

}  // extern "C"
