// Fused sign + im2col + bit-pack + transpose of the activation operand.
//
// Replaces, in one launch and without any float im2col buffer in HBM:
//   c%32==0 ("word path"): repack_input_gpu_bin (src-lib/im2col_kernels.cu:679-724) -> im2col_ongpu (:33-89)
//                          -> transpose_uint32_gpu (:523-549); CPU: src-lib/gemm.cpp:2202-2239 + im2col
//   otherwise ("bit path"): im2col_align_ongpu (:93-154) -> float_to_bit_gpu (:285-317) -> transpose_bin_gpu
//                          (:424-520); CPU: im2col_cpu_custom_bin + transpose_bin (src-lib/gemm.cpp:1339-1460, :216-245)
// and writes the reference's t_bit_input layout: row (b*N + p) = the K sign bits of output pixel p of
// image b, followed by zero padding up to new_ldb bits.
//
// Structure of both kernels: one CTA owns a strip of output rows of one image.
//   phase A  reads the fp32 input rows the strip needs exactly once, coalesced (float4 where the row
//            pitch allows), and leaves sign bits in shared memory (32 channels per word on the word
//            path; one bit plane per channel, built with __ballot_sync, on the bit path);
//   phase B  assembles complete rows of the packed operand from shared memory and stores them with
//            16-byte writes, so global stores are contiguous along K.
// HBM traffic per image is therefore 4*C*H*W bytes read (plus halo rows, served by L2) and
// N*new_ldb/8 bytes written.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int PK_THREADS = 256;
constexpr size_t PK_MAX_SMEM = 200 * 1024;

struct PackParams
{
	const float * in;
	uint32_t * out;
	int C, H, W, OH, OW;
	int ks, stride, pad;
	int rows_per_cta;    // output rows per CTA
	int tiles_per_image;
	int ldw;             // words per packed row (new_ldb/32)
	int K;               // bits per row that carry data
	int max_in_rows;     // input rows a strip can touch
};

// ---- word path -----------------------------------------------------------------------------
// shared: packed[CB][R][W] words, CB = C/32, R = input rows of this strip.
template <bool VEC4>
__global__ void __launch_bounds__(PK_THREADS)
pack_input_words_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int b = blockIdx.x / p.tiles_per_image;
	const int tile = blockIdx.x - b * p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int iy_lo = max(y0 * p.stride - p.pad, 0);
	const int iy_hi = min((y1 - 1) * p.stride - p.pad + p.ks - 1, p.H - 1);
	const int R = iy_hi - iy_lo + 1;          // may be <= 0 when the strip only sees padding
	const int CB = p.C >> 5;
	const int span = max(R, 0) * p.W;         // contiguous floats per channel
	const size_t chan_stride = (size_t)p.H * p.W;
	const float * img = p.in + (size_t)b * p.C * chan_stride + (size_t)iy_lo * p.W;

	// phase A: 32 channels -> one word per input pixel
	if (VEC4)
	{
		const int span4 = span >> 2;
		for (int idx = threadIdx.x; idx < CB * span4; idx += PK_THREADS)
		{
			const int cb = idx / span4;
			const int e4 = idx - cb * span4;
			const float4 * src = reinterpret_cast<const float4 *>(img + (size_t)cb * 32 * chan_stride) + e4;
			uint32_t w0 = 0, w1 = 0, w2 = 0, w3 = 0;
			#pragma unroll
			for (int ch = 0; ch < 32; ++ch)
			{
				const float4 v = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(src) + (size_t)ch * chan_stride));
				w0 |= (v.x > 0 ? 1u : 0u) << ch;
				w1 |= (v.y > 0 ? 1u : 0u) << ch;
				w2 |= (v.z > 0 ? 1u : 0u) << ch;
				w3 |= (v.w > 0 ? 1u : 0u) << ch;
			}
			reinterpret_cast<uint4 *>(s_words)[idx] = make_uint4(w0, w1, w2, w3);
		}
	}
	else
	{
		for (int idx = threadIdx.x; idx < CB * span; idx += PK_THREADS)
		{
			const int cb = idx / span;
			const int e = idx - cb * span;
			const float * src = img + (size_t)cb * 32 * chan_stride + e;
			uint32_t w0 = 0;
			#pragma unroll
			for (int ch = 0; ch < 32; ++ch)
			{
				w0 |= (__ldg(src + (size_t)ch * chan_stride) > 0 ? 1u : 0u) << ch;
			}
			s_words[idx] = w0;
		}
	}
	__syncthreads();

	// phase B: one uint4 (4 K-words) per thread-iteration
	const int taps = p.ks * p.ks;
	const int new_k = CB * taps;
	const int ldq = p.ldw >> 2;
	const int pixels = (y1 - y0) * p.OW;
	const size_t row_base = (size_t)b * p.OH * p.OW + (size_t)y0 * p.OW;
	for (int q = threadIdx.x; q < pixels * ldq; q += PK_THREADS)
	{
		const int pl = q / ldq;
		const int wq = q - pl * ldq;
		const int yl = pl / p.OW;
		const int x = pl - yl * p.OW;
		const int iy_base = (y0 + yl) * p.stride - p.pad - iy_lo;   // relative to the staged rows
		const int ix_base = x * p.stride - p.pad;
		uint32_t v[4];
		#pragma unroll
		for (int u = 0; u < 4; ++u)
		{
			const int wi = wq * 4 + u;
			uint32_t word = 0;
			if (wi < new_k)
			{
				const int cb = wi / taps;
				const int t = wi - cb * taps;
				const int ky = t / p.ks;
				const int kx = t - ky * p.ks;
				const int r = iy_base + ky;
				const int ix = ix_base + kx;
				if (r >= 0 && r < R && ix >= 0 && ix < p.W) { word = s_words[(cb * R + r) * p.W + ix]; }
			}
			v[u] = word;
		}
		reinterpret_cast<uint4 *>(p.out + (row_base + pl) * p.ldw)[wq] = make_uint4(v[0], v[1], v[2], v[3]);
	}
}

// ---- bit path ------------------------------------------------------------------------------
// shared: planes[C][R][PW] words, PW = ceil(W/32); bit x of plane row (c, r) = input(c, iy_lo+r, x) > 0.
__global__ void __launch_bounds__(PK_THREADS)
pack_input_bits_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int b = blockIdx.x / p.tiles_per_image;
	const int tile = blockIdx.x - b * p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int iy_lo = max(y0 * p.stride - p.pad, 0);
	const int iy_hi = min((y1 - 1) * p.stride - p.pad + p.ks - 1, p.H - 1);
	const int R = max(iy_hi - iy_lo + 1, 0);
	const int PW = (p.W + 31) >> 5;
	const size_t chan_stride = (size_t)p.H * p.W;
	const float * img = p.in + (size_t)b * p.C * chan_stride;

	// phase A: one warp ballot per 32 consecutive pixels of one (channel, row)
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	const int items = p.C * R * PW;
	for (int it = warp; it < items; it += PK_THREADS / 32)
	{
		const int xw = it % PW;
		const int cr = it / PW;
		const int r = cr % R;
		const int c = cr / R;
		const int x = xw * 32 + lane;
		float v = 0.0f;
		if (x < p.W) { v = __ldg(img + (size_t)c * chan_stride + (size_t)(iy_lo + r) * p.W + x); }
		const uint32_t word = __ballot_sync(0xffffffffu, v > 0);
		if (lane == 0) { s_words[it] = word; }
	}
	__syncthreads();

	// phase B: thread builds 4 consecutive K-words of one output row; k = c*taps + ky*ks + kx
	const int taps = p.ks * p.ks;
	const int ldq = p.ldw >> 2;
	const int pixels = (y1 - y0) * p.OW;
	const size_t row_base = (size_t)b * p.OH * p.OW + (size_t)y0 * p.OW;
	for (int q = threadIdx.x; q < pixels * ldq; q += PK_THREADS)
	{
		const int pl = q / ldq;
		const int wq = q - pl * ldq;
		const int yl = pl / p.OW;
		const int x = pl - yl * p.OW;
		const int iy_base = (y0 + yl) * p.stride - p.pad - iy_lo;
		const int ix_base = x * p.stride - p.pad;
		int k = wq * 128;
		int c = k / taps;
		int t = k - c * taps;
		int ky = t / p.ks;
		int kx = t - ky * p.ks;
		uint32_t v[4];
		#pragma unroll
		for (int u = 0; u < 4; ++u)
		{
			uint32_t word = 0;
			for (int bit = 0; bit < 32; ++bit)
			{
				if (k < p.K)
				{
					const int r = iy_base + ky;
					const int ix = ix_base + kx;
					if (r >= 0 && r < R && ix >= 0 && ix < p.W)
					{
						word |= ((s_words[(c * R + r) * PW + (ix >> 5)] >> (ix & 31)) & 1u) << bit;
					}
				}
				++k;
				if (++kx == p.ks) { kx = 0; if (++ky == p.ks) { ky = 0; ++c; } }
			}
			v[u] = word;
		}
		reinterpret_cast<uint4 *>(p.out + (row_base + pl) * p.ldw)[wq] = make_uint4(v[0], v[1], v[2], v[3]);
	}
}

// ---- channel pack only (stage-level seam) -----------------------------------------------------
// input [c][hw] -> packed [c/32][hw]; one thread per output word, coalesced along hw.
__global__ void __launch_bounds__(PK_THREADS)
repack_input_bin_kernel(const float * __restrict__ in, uint32_t * __restrict__ out, int hw, int cb_count)
{
	const size_t total = (size_t)hw * cb_count;
	for (size_t idx = (size_t)blockIdx.x * PK_THREADS + threadIdx.x; idx < total; idx += (size_t)gridDim.x * PK_THREADS)
	{
		const size_t cb = idx / hw;
		const size_t e = idx - cb * hw;
		const float * src = in + cb * 32 * hw + e;
		uint32_t word = 0;
		#pragma unroll
		for (int ch = 0; ch < 32; ++ch) { word |= (__ldg(src + (size_t)ch * hw) > 0 ? 1u : 0u) << ch; }
		out[idx] = word;
	}
}

// fp32 -> sign bits, 32 floats per warp ballot; dst word i covers src[32*i .. 32*i+31].
__global__ void __launch_bounds__(PK_THREADS)
float_to_bit_kernel(const float * __restrict__ src, uint32_t * __restrict__ dst, size_t size)
{
	const size_t words = (size + 31) / 32;
	const int lane = threadIdx.x & 31;
	const size_t warps_total = (size_t)gridDim.x * (PK_THREADS / 32);
	for (size_t w = (size_t)blockIdx.x * (PK_THREADS / 32) + (threadIdx.x >> 5); w < words; w += warps_total)
	{
		const size_t i = w * 32 + lane;
		const float v = (i < size) ? __ldg(src + i) : 0.0f;
		const uint32_t word = __ballot_sync(0xffffffffu, v > 0);
		if (lane == 0) { dst[w] = word; }
	}
}

int launch_pack_input(const xnor_b200_conv_desc & d, const float * input, uint32_t * t_bit_input, cudaStream_t stream)
{
	PackParams p;
	p.in = input;
	p.out = t_bit_input;
	p.C = d.c; p.H = d.h; p.W = d.w;
	p.OH = conv_out_dim(d.h, d.size, d.stride, d.pad);
	p.OW = conv_out_dim(d.w, d.size, d.stride, d.pad);
	p.ks = d.size; p.stride = d.stride; p.pad = d.pad;
	p.K = d.size * d.size * d.c;
	p.ldw = aligned_lda(p.K) / 32;
	const bool word_path = (d.c % 32 == 0);

	// bytes of shared memory per staged input row
	const size_t row_bytes = word_path ? (size_t)(d.c / 32) * d.w * 4 : (size_t)d.c * ((d.w + 31) / 32) * 4;
	auto in_rows = [&](int out_rows) { return (out_rows - 1) * d.stride + d.size; };
	if (row_bytes * (size_t)min(in_rows(1), d.h) > PK_MAX_SMEM) { return XNOR_B200_ERR_TOO_LARGE; }

	// Largest strip that (a) fits shared memory and (b) still leaves about two CTAs per SM.
	const int want_ctas = 2 * sm_count();
	int rows = p.OH;
	while (rows > 1 && (row_bytes * (size_t)min(in_rows(rows), d.h) > PK_MAX_SMEM
			|| (long long)d.batch * ((p.OH + rows - 1) / rows) < want_ctas))
	{
		--rows;
	}
	p.rows_per_cta = rows;
	p.tiles_per_image = (p.OH + rows - 1) / rows;
	p.max_in_rows = min(in_rows(rows), d.h);
	const size_t smem = round_up(row_bytes * (size_t)p.max_in_rows, 16);
	const long long grid = (long long)d.batch * p.tiles_per_image;
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }

	if (word_path)
	{
		const bool vec4 = (d.w % 4 == 0) && (((uintptr_t)input & 15u) == 0);
		auto kern = vec4 ? pack_input_words_kernel<true> : pack_input_words_kernel<false>;
		int rc = ensure_dynamic_smem((const void *)kern, smem > 48 * 1024 ? PK_MAX_SMEM : 0);
		if (rc != XNOR_B200_OK) { return rc; }
		kern<<<(unsigned)grid, PK_THREADS, smem, stream>>>(p);
	}
	else
	{
		int rc = ensure_dynamic_smem((const void *)pack_input_bits_kernel, smem > 48 * 1024 ? PK_MAX_SMEM : 0);
		if (rc != XNOR_B200_OK) { return rc; }
		pack_input_bits_kernel<<<(unsigned)grid, PK_THREADS, smem, stream>>>(p);
	}
	return check_launch();
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_pack_input(const xnor_b200_conv_desc * desc, const float * input, uint8_t * t_bit_input, void * stream)
{
	if (desc == nullptr || input == nullptr || t_bit_input == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (((uintptr_t)t_bit_input & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	return launch_pack_input(*desc, input, (uint32_t *)t_bit_input, (cudaStream_t)stream);
}

extern "C" int xnor_b200_repack_input_bin(const float * input, uint32_t * packed, int w, int h, int c, void * stream)
{
	if (input == nullptr || packed == nullptr) { return XNOR_B200_ERR_NULL; }
	if (w <= 0 || h <= 0 || c <= 0 || c % 32 != 0) { return XNOR_B200_ERR_INVALID; }
	const size_t total = (size_t)w * h * (c / 32);
	const int grid = (int)min((total + PK_THREADS - 1) / PK_THREADS, (size_t)sm_count() * 16);
	repack_input_bin_kernel<<<grid, PK_THREADS, 0, (cudaStream_t)stream>>>(input, packed, w * h, c / 32);
	return check_launch();
}

extern "C" int xnor_b200_float_to_bit(const float * src, uint8_t * dst, size_t size, void * stream)
{
	if (src == nullptr || dst == nullptr) { return XNOR_B200_ERR_NULL; }
	if (size == 0) { return XNOR_B200_ERR_INVALID; }
	if (((uintptr_t)dst & 3u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	const size_t words = (size + 31) / 32;
	const int grid = (int)min((words + 7) / 8, (size_t)sm_count() * 16);
	float_to_bit_kernel<<<grid, PK_THREADS, 0, (cudaStream_t)stream>>>(src, (uint32_t *)dst, size);
	return check_launch();
}
