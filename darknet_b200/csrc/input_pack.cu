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
// Structure of both kernels: one CTA owns a strip of output rows of one image (word path: and a group of
// 32-channel blocks, so that small feature maps still spread over many SMs).
//   phase A  reads the fp32 input rows the strip needs exactly once, coalesced (float4 where the row
//            pitch allows), and leaves sign bits in shared memory: 32 channels per word on the word path
//            (four threads share a word, eight channels each, to keep more loads in flight), one bit plane
//            per channel built with __ballot_sync on the bit path;
//   phase B  assembles the packed rows from shared memory and stores them with 16-byte writes, contiguous
//            along K.  On the bit path a thread pulls `size` adjacent bits of one (channel, kernel row) per
//            step out of a bit plane with a funnel shift instead of testing taps one by one.
// HBM traffic per image is therefore 4*C*H*W bytes read (plus halo rows, served by L2) and
// N*new_ldb/8 bytes written.
#include "xnor_common.cuh"

#include <cstdlib>

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
	int tiles_per_image; // row strips per image
	int cb_per_cta;      // word path: 32-channel blocks per CTA (a multiple of 4 unless it covers all of them)
	int groups;          // word path: channel-block groups per strip
	int ldw;             // words per packed row (new_ldb/32)
	int K;               // bits per row that carry data
};

// ---- word path -----------------------------------------------------------------------------
// shared: packed[cb_local][R][W] words, R = input rows of this strip.
// VEC  = floats per load (4, 2 or 1, as the row pitch and pointer alignment allow);
// SUBS = threads sharing one output word, each covering 32/SUBS channels (4 on small problems, to put more threads
//        to work; 1 on large ones, where a thread then keeps 32 independent loads in flight).
template <int VEC, int SUBS>
__global__ void __launch_bounds__(PK_THREADS)
pack_input_words_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int g = blockIdx.x % p.groups;
	const int rest = blockIdx.x / p.groups;
	const int tile = rest % p.tiles_per_image;
	const int b = rest / p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int iy_lo = max(y0 * p.stride - p.pad, 0);
	const int iy_hi = min((y1 - 1) * p.stride - p.pad + p.ks - 1, p.H - 1);
	const int R = iy_hi - iy_lo + 1;          // may be <= 0 when the strip only sees padding
	const int CB = p.C >> 5;
	const int cb0 = g * p.cb_per_cta;
	const int cbn = min(p.cb_per_cta, CB - cb0);
	const int span = max(R, 0) * p.W;         // contiguous floats per channel
	const size_t chan_stride = (size_t)p.H * p.W;
	const float * img = p.in + ((size_t)b * p.C + (size_t)cb0 * 32) * chan_stride + (size_t)iy_lo * p.W;

	// phase A: 32 channels -> one word per input pixel
	{
		constexpr int CH = 32 / SUBS;             // channels per thread-task
		const int spanv = span / VEC;             // VEC divides W, hence span
		const int items = cbn * spanv;
		for (int idx = threadIdx.x; idx < items * SUBS; idx += PK_THREADS)
		{
			const int sub = idx / items;
			const int item = idx - sub * items;
			const int cbl = item / spanv;
			const int ev = item - cbl * spanv;
			const float * src = img + ((size_t)cbl * 32 + sub * CH) * chan_stride + (size_t)ev * VEC;
			uint32_t w[VEC];
			#pragma unroll
			for (int j = 0; j < VEC; ++j) { w[j] = 0; }
			#pragma unroll
			for (int ch = 0; ch < CH; ++ch)
			{
				const float * q = src + (size_t)ch * chan_stride;
				if (VEC == 4)
				{
					const float4 v = __ldg(reinterpret_cast<const float4 *>(q));
					w[0] |= (v.x > 0 ? 1u : 0u) << ch;
					w[1 % VEC] |= (v.y > 0 ? 1u : 0u) << ch;
					w[2 % VEC] |= (v.z > 0 ? 1u : 0u) << ch;
					w[3 % VEC] |= (v.w > 0 ? 1u : 0u) << ch;
				}
				else if (VEC == 2)
				{
					const float2 v = __ldg(reinterpret_cast<const float2 *>(q));
					w[0] |= (v.x > 0 ? 1u : 0u) << ch;
					w[1 % VEC] |= (v.y > 0 ? 1u : 0u) << ch;
				}
				else
				{
					w[0] |= (__ldg(q) > 0 ? 1u : 0u) << ch;
				}
			}
			if (SUBS == 1)
			{
				#pragma unroll
				for (int j = 0; j < VEC; ++j) { s_words[(size_t)item * VEC + j] = w[j]; }
			}
			else
			{
				// SUBS == 4: this thread owns byte `sub` of each word
				uint8_t * dst = reinterpret_cast<uint8_t *>(s_words) + (size_t)item * VEC * 4 + sub;
				#pragma unroll
				for (int j = 0; j < VEC; ++j) { dst[j * 4] = (uint8_t)w[j]; }
			}
		}
	}
	__syncthreads();

	// phase B: one uint4 (4 K-words) per thread-iteration over this CTA's word range
	const int taps = p.ks * p.ks;
	const int new_k = CB * taps;
	const bool last_group = (g == p.groups - 1);
	const int q_lo = (cb0 * taps) >> 2;                                   // cb0 % 4 == 0 whenever groups > 1
	const int q_hi = last_group ? (p.ldw >> 2) : (((cb0 + cbn) * taps) >> 2);
	const int nq = q_hi - q_lo;
	const int pixels = (y1 - y0) * p.OW;
	const size_t row_base = (size_t)b * p.OH * p.OW + (size_t)y0 * p.OW;
	for (int q = threadIdx.x; q < pixels * nq; q += PK_THREADS)
	{
		const int pl = q / nq;
		const int wq = q_lo + (q - pl * nq);
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
				if (r >= 0 && r < R && ix >= 0 && ix < p.W) { word = s_words[((cb - cb0) * R + r) * p.W + ix]; }
			}
			v[u] = word;
		}
		reinterpret_cast<uint4 *>(p.out + (row_base + pl) * p.ldw)[wq] = make_uint4(v[0], v[1], v[2], v[3]);
	}
}

// ---- bit path ------------------------------------------------------------------------------
// shared: planes[C][RR][PW] words.  Row rr of a strip is input row y0*stride - pad + rr (rows outside the image
// are all zero); bit (ix + pad) of a plane row = input(c, row, ix) > 0, so the `ks` taps of one kernel row of
// output column x are the adjacent bits x*stride .. x*stride + ks - 1.  PW has one spare word for the funnel shift.
__global__ void __launch_bounds__(PK_THREADS)
pack_input_bits_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int tile = blockIdx.x % p.tiles_per_image;
	const int b = blockIdx.x / p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int RR = (y1 - y0 - 1) * p.stride + p.ks;
	const int PW = ((p.W + 2 * p.pad + 31) >> 5) + 1;
	const size_t chan_stride = (size_t)p.H * p.W;
	const float * img = p.in + (size_t)b * p.C * chan_stride;
	const int iy0 = y0 * p.stride - p.pad;

	// phase A: one warp ballot per 32 consecutive padded positions of one (channel, row)
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	const int items = p.C * RR * PW;
	constexpr int NWARPS = PK_THREADS / 32;
	constexpr int UNROLL = 8;                              // loads in flight per lane before the first ballot
	for (int base = warp; base < items; base += UNROLL * NWARPS)
	{
		float v[UNROLL];
		#pragma unroll
		for (int u = 0; u < UNROLL; ++u)
		{
			const int it = base + u * NWARPS;
			const int xw = it % PW;
			const int cr = it / PW;
			const int rr = cr % RR;
			const int c = cr / RR;
			const int ix = xw * 32 + lane - p.pad;
			const int iy = iy0 + rr;
			v[u] = 0.0f;
			if (it < items && ix >= 0 && ix < p.W && iy >= 0 && iy < p.H)
			{
				v[u] = __ldg(img + (size_t)c * chan_stride + (size_t)iy * p.W + ix);
			}
		}
		#pragma unroll
		for (int u = 0; u < UNROLL; ++u)
		{
			const int it = base + u * NWARPS;
			const uint32_t word = __ballot_sync(0xffffffffu, v[u] > 0);
			if (lane == 0 && it < items) { s_words[it] = word; }
		}
	}
	__syncthreads();

	// phase B: thread builds 4 consecutive K-words (bits k0 .. k0+127) of one output row.
	// K order: k = (c*ks + ky)*ks + kx, i.e. consecutive groups (c, ky) of ks bits each.
	const int ldq = p.ldw >> 2;
	const int pixels = (y1 - y0) * p.OW;
	const int n_groups = p.C * p.ks;
	const uint32_t tap_mask = (p.ks >= 32) ? 0xffffffffu : ((1u << p.ks) - 1u);
	const size_t row_base = (size_t)b * p.OH * p.OW + (size_t)y0 * p.OW;
	for (int q = threadIdx.x; q < pixels * ldq; q += PK_THREADS)
	{
		const int pl = q / ldq;
		const int wq = q - pl * ldq;
		const int yl = pl / p.OW;
		const int x = pl - yl * p.OW;
		const int p0 = x * p.stride;                       // first tap, in padded plane coordinates
		const int sh = p0 & 31;
		const int k0 = wq * 128;
		int grp = k0 / p.ks;
		int skip = k0 - grp * p.ks;                        // bits of the first group that belong to the previous quad
		int c = grp / p.ks;
		int ky = grp - c * p.ks;
		const uint32_t * plane = s_words + ((size_t)c * RR + (size_t)yl * p.stride) * PW + (p0 >> 5);
		uint32_t v[4] = {0u, 0u, 0u, 0u};
		unsigned long long buf = 0ull;
		int fill = 0, outw = 0;
		while (outw < 4 && grp < n_groups)
		{
			const uint32_t * row = plane + ky * PW;
			uint32_t bits = __funnelshift_r(row[0], row[1], sh) & tap_mask;
			bits >>= skip;
			buf |= (unsigned long long)bits << fill;
			fill += p.ks - skip;
			skip = 0;
			if (fill >= 32)
			{
				v[outw++] = (uint32_t)buf;
				buf >>= 32;
				fill -= 32;
			}
			++grp;
			if (++ky == p.ks) { ky = 0; plane += (size_t)RR * PW; }
		}
		if (outw < 4 && fill > 0) { v[outw] = (uint32_t)buf; }
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
	// CTAs to aim for.  Each CTA loads, synchronises, then stores, so overlap of loads and stores comes from
	// several CTAs sharing an SM.  XNOR_B200_PACK_CTAS_PER_SM overrides the factor (tuning aid).
	int ctas_per_sm = 4;
	if (const char * e = std::getenv("XNOR_B200_PACK_CTAS_PER_SM")) { ctas_per_sm = max(1, atoi(e)); }
	const int want_ctas = ctas_per_sm * sm_count();
	auto in_rows = [&](int out_rows) { return (out_rows - 1) * d.stride + d.size; };

	if (word_path)
	{
		const int CB = d.c / 32;
		// Parallelism is taken in order of cost: images (free), then groups of 32-channel blocks (free, no halo;
		// group borders stay on multiples of 4 blocks so that every group's word range starts on a 16-byte
		// boundary of the packed row), then row strips (each strip re-reads size-1 halo rows).
		long long ctas = d.batch;
		int cb_per_cta = CB;
		if (ctas < want_ctas && CB >= 8)
		{
			const int groups = (int)min((long long)(CB / 4), (want_ctas + ctas - 1) / ctas);
			cb_per_cta = (int)round_up((size_t)(CB + groups - 1) / groups, 4);
		}
		p.cb_per_cta = cb_per_cta;
		p.groups = (CB + cb_per_cta - 1) / cb_per_cta;
		ctas *= p.groups;
		const size_t row_bytes = (size_t)cb_per_cta * d.w * 4;
		if (row_bytes * (size_t)min(in_rows(1), d.h) > PK_MAX_SMEM) { return XNOR_B200_ERR_TOO_LARGE; }
		const int strips = (int)min((long long)p.OH, max(1LL, (want_ctas + ctas - 1) / ctas));
		int rows = (p.OH + strips - 1) / strips;
		while (rows > 1 && row_bytes * (size_t)min(in_rows(rows), d.h) > PK_MAX_SMEM) { --rows; }
		p.rows_per_cta = rows;
		p.tiles_per_image = (p.OH + rows - 1) / rows;
		const size_t smem = round_up(row_bytes * (size_t)min(in_rows(rows), d.h), 16);
		const long long grid = (long long)d.batch * p.tiles_per_image * p.groups;
		if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
		const int vec = ((d.w % 4 == 0) && (((uintptr_t)input & 15u) == 0)) ? 4
				: ((d.w % 2 == 0) && (((uintptr_t)input & 7u) == 0)) ? 2 : 1;
		// words per CTA in phase A; below two per thread the channel split keeps more threads busy
		const long long words_per_cta = (long long)cb_per_cta * min(in_rows(rows), d.h) * d.w;
		const bool split = words_per_cta < 2LL * PK_THREADS * vec;
		void (*kern)(const PackParams) =
				vec == 4 ? (split ? pack_input_words_kernel<4, 4> : pack_input_words_kernel<4, 1>)
				: vec == 2 ? (split ? pack_input_words_kernel<2, 4> : pack_input_words_kernel<2, 1>)
				: (split ? pack_input_words_kernel<1, 4> : pack_input_words_kernel<1, 1>);
		int rc = ensure_dynamic_smem((const void *)kern, smem > 48 * 1024 ? PK_MAX_SMEM : 0);
		if (rc != XNOR_B200_OK) { return rc; }
		kern<<<(unsigned)grid, PK_THREADS, smem, stream>>>(p);
	}
	else
	{
		if (d.size > 24) { return XNOR_B200_ERR_TOO_LARGE; }      // a kernel row must fit the 64-bit assembly buffer
		p.cb_per_cta = 0;
		p.groups = 1;
		const int PW = ((d.w + 2 * d.pad + 31) >> 5) + 1;
		const size_t row_bytes = (size_t)d.c * PW * 4;
		if (row_bytes * (size_t)in_rows(1) > PK_MAX_SMEM) { return XNOR_B200_ERR_TOO_LARGE; }
		int rows = p.OH;
		while (rows > 1 && (row_bytes * (size_t)in_rows(rows) > PK_MAX_SMEM
				|| (long long)d.batch * ((p.OH + rows - 1) / rows) < want_ctas))
		{
			--rows;
		}
		p.rows_per_cta = rows;
		p.tiles_per_image = (p.OH + rows - 1) / rows;
		const size_t smem = round_up(row_bytes * (size_t)in_rows(rows), 16);
		const long long grid = (long long)d.batch * p.tiles_per_image;
		if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
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
