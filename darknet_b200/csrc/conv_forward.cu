// Per-layer entry point and shared host-side helpers of the xnor_b200 C ABI.
//
// xnor_b200_conv_forward stands in for the xnor branch of forward_convolutional_layer_gpu
// (src-lib/convolutional_kernels.cu:204-262): two launches per layer (pack, GEMM+epilogue) instead of the
// reference's four, for every image of the batch instead of image 0 only.
#include "xnor_common.cuh"

#include <mutex>
#include <vector>

namespace xnor
{

thread_local int g_last_cuda_error = 0;

static xnor_b200_tuning g_tuning = {};

const xnor_b200_tuning & tuning() { return g_tuning; }

int sm_count()
{
	static int cached[64] = {0};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { return 148; }
	if (cached[dev] == 0)
	{
		int n = 0;
		if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { n = 148; }
		cached[dev] = n;
	}
	return cached[dev];
}

int ensure_dynamic_smem(const void * kernel, size_t bytes)
{
	if (bytes <= 48 * 1024) { return XNOR_B200_OK; }
	struct Entry { const void * kernel; int device; size_t bytes; };
	static std::mutex mu;
	static std::vector<Entry> done;
	int dev = 0;
	cudaError_t e = cudaGetDevice(&dev);
	if (e != cudaSuccess) { return cuda_fail(e); }
	std::lock_guard<std::mutex> lock(mu);
	for (Entry & en : done)
	{
		if (en.kernel == kernel && en.device == dev)
		{
			if (en.bytes >= bytes) { return XNOR_B200_OK; }
			e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
			if (e != cudaSuccess) { return cuda_fail(e); }
			en.bytes = bytes;
			return XNOR_B200_OK;
		}
	}
	e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
	if (e != cudaSuccess) { return cuda_fail(e); }
	done.push_back({kernel, dev, bytes});
	return XNOR_B200_OK;
}

int validate_desc(const xnor_b200_conv_desc * d)
{
	if (d->batch <= 0 || d->c <= 0 || d->h <= 0 || d->w <= 0 || d->n <= 0) { return XNOR_B200_ERR_INVALID; }
	if (d->size <= 0 || d->stride <= 0 || d->pad < 0) { return XNOR_B200_ERR_INVALID; }
	if (d->activation != XNOR_B200_LINEAR && d->activation != XNOR_B200_LEAKY) { return XNOR_B200_ERR_INVALID; }
	if (d->h + 2 * d->pad < d->size || d->w + 2 * d->pad < d->size) { return XNOR_B200_ERR_INVALID; }
	// Everything below is indexed with 32-bit ints inside the kernels.
	const long long k = (long long)d->size * d->size * d->c;
	const long long n_out = (long long)conv_out_dim(d->h, d->size, d->stride, d->pad) * conv_out_dim(d->w, d->size, d->stride, d->pad);
	if (k > (1 << 24) || n_out * d->batch > 0x7fffffffLL - 1024 || (long long)d->c * d->h * d->w > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	return XNOR_B200_OK;
}

}  // namespace xnor

using namespace xnor;

extern "C" const char * xnor_b200_strerror(int code)
{
	switch (code)
	{
		case XNOR_B200_OK:            return "ok";
		case XNOR_B200_ERR_INVALID:   return "invalid size, stride or enum argument";
		case XNOR_B200_ERR_NULL:      return "required pointer is NULL";
		case XNOR_B200_ERR_SCRATCH:   return "scratch buffer too small";
		case XNOR_B200_ERR_CUDA:      return "CUDA runtime call failed";
		case XNOR_B200_ERR_ALIGNMENT: return "pointer or leading dimension not aligned";
		case XNOR_B200_ERR_TOO_LARGE: return "size exceeds a fixed limit of this entry point";
		default:                      return "unknown xnor_b200 error code";
	}
}

extern "C" int xnor_b200_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int xnor_b200_set_tuning(const xnor_b200_tuning * t)
{
	if (t == nullptr)
	{
		g_tuning = xnor_b200_tuning();
		return XNOR_B200_OK;
	}
	if (t->gemm_route < XNOR_B200_ROUTE_AUTO || t->gemm_route > XNOR_B200_ROUTE_TILED) { return XNOR_B200_ERR_INVALID; }
	if (t->gemm_tile < 0 || t->gemm_split < 0 || t->gemm_split > 8 || t->pack_ctas_per_sm < 0 || t->pack_ctas_per_sm > 32) { return XNOR_B200_ERR_INVALID; }
	if (t->pack_two_pass < 0 || t->pack_two_pass > 2) { return XNOR_B200_ERR_INVALID; }
	if (t->tc_kernel < 0 || t->tc_kernel > 2) { return XNOR_B200_ERR_INVALID; }
	if (t->tc_wait_polls < 0 || t->tc_withhold_arrival < 0 || t->tc_withhold_arrival > 1) { return XNOR_B200_ERR_INVALID; }
	g_tuning = *t;
	return XNOR_B200_OK;
}

extern "C" int xnor_b200_take_device_status(int * status)
{
	if (status == nullptr) { return XNOR_B200_ERR_NULL; }
	cudaError_t e = cudaDeviceSynchronize();
	if (e != cudaSuccess) { return cuda_fail(e); }
	return read_tc_error(status, true);
}

extern "C" int xnor_b200_conv_geometry(const xnor_b200_conv_desc * desc, xnor_b200_conv_geom * geom)
{
	if (desc == nullptr || geom == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	geom->out_h = conv_out_dim(desc->h, desc->size, desc->stride, desc->pad);
	geom->out_w = conv_out_dim(desc->w, desc->size, desc->stride, desc->pad);
	geom->n_out = geom->out_h * geom->out_w;
	geom->k = desc->size * desc->size * desc->c;
	geom->new_lda = aligned_lda(geom->k);
	geom->bit_align = aligned_n(geom->n_out);
	geom->word_path = (desc->c % 32 == 0) ? 1 : 0;
	geom->weights_bytes = (size_t)desc->n * geom->new_lda / 8;
	geom->packed_input_bytes = (size_t)desc->batch * geom->n_out * geom->new_lda / 8;
	geom->output_floats = (size_t)desc->batch * desc->n * geom->n_out;
	return XNOR_B200_OK;
}

extern "C" size_t xnor_b200_scratch_bytes(const xnor_b200_conv_desc * desc)
{
	xnor_b200_conv_geom g;
	if (xnor_b200_conv_geometry(desc, &g) != XNOR_B200_OK) { return 0; }
	return round_up(g.packed_input_bytes, 256);
}

// Fills the kernel-side description of one sign sink; checks that the tensor this layer produces (after the optional
// pool / upsample) is exactly the consumer's input.
static int make_sink(const xnor_b200_conv_desc * desc, const xnor_b200_conv_geom & g, const xnor_b200_sign_sink & in, SinkParams * out)
{
	const xnor_b200_conv_desc * c = in.consumer;
	if (c == nullptr || in.consumer_scratch == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(c);
	if (rc != XNOR_B200_OK) { return rc; }
	if (c->c % 32 != 0 || c->stride != 1 || 2 * c->pad != c->size - 1 || c->batch != desc->batch) { return XNOR_B200_ERR_INVALID; }
	if (in.channel_offset < 0 || in.channel_offset % 32 != 0 || in.channel_offset + desc->n > c->c) { return XNOR_B200_ERR_INVALID; }
	if ((in.pool != 0 && in.pool != 2) || (in.upsample != 0 && in.upsample != 1 && in.upsample != 2)) { return XNOR_B200_ERR_INVALID; }
	if (in.pool == 2 && in.upsample == 2) { return XNOR_B200_ERR_INVALID; }
	int h = g.out_h, w = g.out_w;
	if (in.pool == 2)
	{
		if (h % 2 != 0 || w % 2 != 0) { return XNOR_B200_ERR_INVALID; }
		h /= 2; w /= 2;
	}
	if (in.upsample == 2) { h *= 2; w *= 2; }
	if (h != c->h || w != c->w) { return XNOR_B200_ERR_INVALID; }
	if (in.consumer_window_major && (c->h % 2 != 0 || c->w % 2 != 0)) { return XNOR_B200_ERR_INVALID; }
	if ((((uintptr_t)in.consumer_scratch) & 255u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	out->operand = (uint32_t *)in.consumer_scratch;
	out->ldw = aligned_lda(c->size * c->size * c->c) / 32;
	out->out_h = c->h; out->out_w = c->w; out->n_out = c->h * c->w;
	out->ks = c->size; out->pad = c->pad; out->taps = c->size * c->size;
	out->cb_offset = in.channel_offset / 32;
	out->pool = in.pool;
	out->up = (in.upsample == 2) ? 2 : 1;
	out->win_w = in.consumer_window_major ? c->w / 2 : 0;
	return XNOR_B200_OK;
}

static int conv_forward_impl(const xnor_b200_conv_desc * desc, const xnor_b200_conv_io & io,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		void * scratch, size_t scratch_bytes, void * stream)
{
	if (desc == nullptr || align_bit_weights == nullptr || mean_arr == nullptr || scratch == nullptr) { return XNOR_B200_ERR_NULL; }
	const int n_in = (io.input != nullptr) + (io.input_signs != nullptr) + (io.input_packed != 0) + (io.input_masks != nullptr);
	if (n_in != 1) { return XNOR_B200_ERR_NULL; }
	if (io.n_sinks < 0 || io.n_sinks > 2 || (io.n_sinks > 0 && io.sinks == nullptr)) { return XNOR_B200_ERR_INVALID; }
	if (io.output != nullptr && io.output_signs != nullptr) { return XNOR_B200_ERR_INVALID; }
	if (io.output == nullptr && io.output_signs == nullptr && io.n_sinks == 0 && io.shortcut_out == nullptr) { return XNOR_B200_ERR_NULL; }
	if ((io.output_signs != nullptr || io.n_sinks > 0) && desc->n % 32 != 0) { return XNOR_B200_ERR_INVALID; }
	if (io.output_signs != nullptr && io.shortcut_out != nullptr) { return XNOR_B200_ERR_INVALID; }
	if (io.input_signs != nullptr && desc->c % 32 != 0 && io.pool != nullptr) { return XNOR_B200_ERR_INVALID; }
	if (io.input_packed && io.pool != nullptr) { return XNOR_B200_ERR_INVALID; }
	xnor_b200_conv_geom g;
	int rc = xnor_b200_conv_geometry(desc, &g);
	if (rc != XNOR_B200_OK) { return rc; }
	if (scratch_bytes < round_up(g.packed_input_bytes, 256)) { return XNOR_B200_ERR_SCRATCH; }
	if ((((uintptr_t)scratch) & 255u) != 0 || (((uintptr_t)align_bit_weights) & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	if (io.shortcut_out != nullptr && io.shortcut_in == nullptr) { return XNOR_B200_ERR_NULL; }
	// the layer's own tensor may be left out when only the fused shortcut sum is wanted -- not together with sign outputs
	if (io.shortcut_out != nullptr && io.output == nullptr && (io.n_sinks > 0 || io.output_signs != nullptr)) { return XNOR_B200_ERR_INVALID; }
	if (io.window_major && (g.out_h % 2 != 0 || g.out_w % 2 != 0)) { return XNOR_B200_ERR_INVALID; }

	GemmExtra extra = GemmExtra();
	extra.win_w = io.window_major ? g.out_w / 2 : 0;
	extra.out_w = g.out_w;
	extra.n_sinks = io.n_sinks;
	for (int i = 0; i < io.n_sinks; ++i)
	{
		rc = make_sink(desc, g, io.sinks[i], &extra.sinks[i]);
		if (rc != XNOR_B200_OK) { return rc; }
		if (io.sinks[i].pool == 2 && !io.window_major) { return XNOR_B200_ERR_INVALID; }
	}

	cudaStream_t s = (cudaStream_t)stream;
	// First xnor layer fed with sign planes, short rows, small problem: the GEMM builds its rows from the planes itself.
	const bool rows_from_planes = (io.input_signs != nullptr && desc->c % 32 != 0
			&& gemm_takes_planes(desc->n, desc->batch * g.n_out, desc->c, desc->size, desc->stride, desc->pad));
	if (io.input_masks != nullptr)
	{
		// channel masks + tap-major weights: only the short-K kernel reads them
		if (!xnor_b200_conv_takes_masks(desc) || !io.tap_major_weights || io.pool != nullptr) { return XNOR_B200_ERR_INVALID; }
		extra.masks = io.input_masks;
		extra.pl_c = desc->c; extra.pl_h = desc->h; extra.pl_w = desc->w;
	}
	else if (rows_from_planes)
	{
		extra.planes = io.input_signs;
		extra.pl_c = desc->c; extra.pl_h = desc->h; extra.pl_w = desc->w;
	}
	else if (!io.input_packed)
	{
		rc = (io.input_signs != nullptr)
				? launch_pack_input(*desc, io.pool, reinterpret_cast<const float *>(io.input_signs), (uint32_t *)scratch, s, 1, io.window_major)
				: launch_pack_input(*desc, io.pool, io.input, (uint32_t *)scratch, s, 0, io.window_major);
		if (rc != XNOR_B200_OK) { return rc; }
	}
	if (io.shortcut_signs != nullptr)
	{
		if (io.shortcut_out == nullptr || desc->n % 32 != 0 || io.n_sinks > 0 || io.output_signs != nullptr) { return XNOR_B200_ERR_INVALID; }
		extra.sum_signs = io.shortcut_signs;
	}
	if (io.shortcut_sink != nullptr)
	{
		// the reader of the fused sum: a 1x1 / stride-1 xnor layer over exactly this layer's filters on the same map
		const xnor_b200_sign_sink & sk = *io.shortcut_sink;
		if (sk.consumer == nullptr || sk.consumer_scratch == nullptr) { return XNOR_B200_ERR_NULL; }
		const xnor_b200_conv_desc & cd = *sk.consumer;
		if (io.shortcut_out == nullptr || desc->n % 32 != 0 || io.n_sinks > 0 || io.output_signs != nullptr || io.window_major) { return XNOR_B200_ERR_INVALID; }
		if (cd.size != 1 || cd.stride != 1 || cd.pad != 0 || cd.c != desc->n || cd.h != g.out_h || cd.w != g.out_w || cd.batch != desc->batch
				|| sk.channel_offset != 0 || sk.pool != 0 || sk.upsample > 1 || sk.consumer_window_major != 0) { return XNOR_B200_ERR_INVALID; }
		if ((((uintptr_t)sk.consumer_scratch) & 255u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
		xnor_b200_conv_geom cg;
		rc = xnor_b200_conv_geometry(&cd, &cg);
		if (rc != XNOR_B200_OK) { return rc; }
		extra.sum_rows = (uint32_t *)sk.consumer_scratch;
		extra.sum_ldw = cg.new_lda / 32;
	}
	const bool extras = (extra.win_w > 0 || extra.n_sinks > 0 || extra.planes != nullptr || extra.masks != nullptr || extra.sum_signs != nullptr
			|| extra.sum_rows != nullptr);
	return launch_xnor_gemm(desc->n, desc->batch * g.n_out, g.n_out, g.k,
			(const uint32_t *)align_bit_weights, g.new_lda / 32, (const uint32_t *)scratch, g.new_lda / 32,
			io.output, g.n_out, mean_arr, biases, desc->activation == XNOR_B200_LEAKY,
			io.shortcut_in, io.shortcut_out, nullptr, s, io.output_signs, extras ? &extra : nullptr);
}

extern "C" int xnor_b200_conv_takes_masks(const xnor_b200_conv_desc * desc)
{
	if (desc == nullptr || validate_desc(desc) != XNOR_B200_OK) { return 0; }
	const int n_out = conv_out_dim(desc->h, desc->size, desc->stride, desc->pad) * conv_out_dim(desc->w, desc->size, desc->stride, desc->pad);
	return ((desc->c == 8 || desc->c == 16)
			&& gemm_takes_planes(desc->n, desc->batch * n_out, desc->c, desc->size, desc->stride, desc->pad)) ? 1 : 0;
}

static xnor_b200_conv_io plain_io(const float * input, const xnor_b200_pool_desc * pool, float * output,
		const float * shortcut_in, float * shortcut_out)
{
	xnor_b200_conv_io io = {};
	io.input = input;
	io.pool = pool;
	io.output = output;
	io.shortcut_in = shortcut_in;
	io.shortcut_out = shortcut_out;
	return io;
}

extern "C" int xnor_b200_conv_forward_io(const xnor_b200_conv_desc * desc, const xnor_b200_conv_io * io,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		void * scratch, size_t scratch_bytes, void * stream)
{
	if (io == nullptr) { return XNOR_B200_ERR_NULL; }
	return conv_forward_impl(desc, *io, align_bit_weights, mean_arr, biases, scratch, scratch_bytes, stream);
}

extern "C" int xnor_b200_conv_forward(const xnor_b200_conv_desc * desc, const float * input,
		const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		float * output, const float * shortcut_in, float * shortcut_out,
		void * scratch, size_t scratch_bytes, void * stream)
{
	if (input == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	return conv_forward_impl(desc, plain_io(input, nullptr, output, shortcut_in, shortcut_out), align_bit_weights, mean_arr, biases,
			scratch, scratch_bytes, stream);
}

extern "C" int xnor_b200_conv_forward_pooled(const xnor_b200_conv_desc * desc, const xnor_b200_pool_desc * pool,
		const float * input, const uint8_t * align_bit_weights, const float * mean_arr, const float * biases,
		float * output, const float * shortcut_in, float * shortcut_out,
		void * scratch, size_t scratch_bytes, void * stream)
{
	if (pool == nullptr) { return XNOR_B200_ERR_NULL; }
	if (input == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	return conv_forward_impl(desc, plain_io(input, pool, output, shortcut_in, shortcut_out), align_bit_weights, mean_arr, biases,
			scratch, scratch_bytes, stream);
}
