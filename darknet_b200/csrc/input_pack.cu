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
	// Optional max-pool in front of the convolution (pool_size == 0: none).  H and W above are then the POOLED
	// sizes the convolution sees, in_h and in_w the sizes of the tensor actually in memory.
	int pool_size, pool_stride, pool_off;
	int in_h, in_w;
	int pool_fast;       // 2x2 window, stride 2, origin 0, even in_h/in_w, 8-byte aligned planes: two float2 loads
	int win_w;           // > 0: output rows of an image in 2x2-window-major pixel order (OW / 2), see out_row()
	int from_planes;     // bit path: `in` holds sign planes uint32 [image][C][H][ceil(W/32)] (bit x%32 of word x/32) instead of floats
	// word path: reciprocals for fast_div() of the divisors the kernels meet, made once on the host
	uint32_t m_ow, m_wp, m_taps, m_ks, m_groups, m_tiles;
	uint32_t m_nq[2];    // threads per pixel in phase B = min(uint4 per pixel of a group, PK_THREADS): [0] every group but the last, [1] the last
	uint32_t m_rv[2];    // staged rows of a strip: [0] full strips, [1] the last (shorter) strip of an image
};

// n / d for 0 <= n < 2^32 / d with m = ceil(2^32 / d): one multiply instead of a division sequence.
__device__ __forceinline__ int fast_div(int n, int d, uint32_t m) { return (d == 1) ? n : (int)__umulhi((uint32_t)n, m); }
static uint32_t div_magic(int d) { return (d <= 1) ? 0u : (uint32_t)(0xffffffffu / (uint32_t)d + 1u); }

// Row of the packed operand that belongs to output pixel (oy, ox) of image b.  Row-major by default; window-major
// (the four pixels of a 2x2 pool window on consecutive rows) when the layer's GEMM epilogue pools its output.
__device__ __forceinline__ size_t out_row(const PackParams & p, int b, int oy, int ox)
{
	const size_t img = (size_t)b * p.OH * p.OW;
	if (p.win_w > 0) { return img + ((size_t)(oy >> 1) * p.win_w + (ox >> 1)) * 4 + (oy & 1) * 2 + (ox & 1); }
	return img + (size_t)oy * p.OW + ox;
}

// sign(maxpool(x)) at pooled position (iy, ix) of one channel plane: the maximum is > 0 exactly when some
// in-image window element is > 0 (window origin -pad/2, out-of-image elements ignored:
// src-lib/maxpool_layer_kernels.cu:48-86), so no maximum is ever formed.
__device__ __forceinline__ bool pooled_positive(const float * __restrict__ plane, const PackParams & p, int iy, int ix)
{
	if (p.pool_fast)
	{
		const float2 * r0 = reinterpret_cast<const float2 *>(plane + (size_t)(2 * iy) * p.in_w) + ix;
		const float2 a = __ldg(r0);
		const float2 c = __ldg(r0 + (p.in_w >> 1));
		return (a.x > 0) || (a.y > 0) || (c.x > 0) || (c.y > 0);
	}
	const int py0 = iy * p.pool_stride - p.pool_off;
	const int px0 = ix * p.pool_stride - p.pool_off;
	bool pos = false;
	for (int l = 0; l < p.pool_size; ++l)
	{
		const int yy = py0 + l;
		if (yy < 0 || yy >= p.in_h) { continue; }
		for (int m = 0; m < p.pool_size; ++m)
		{
			const int xx = px0 + m;
			if (xx >= 0 && xx < p.in_w) { pos = pos || (__ldg(plane + (size_t)yy * p.in_w + xx) > 0); }
		}
	}
	return pos;
}

// Staging layout of the word path, shared by the kernels below: s_words[cbl][RV][WP], the strip's input rows WITH the
// convolution's zero padding written out -- RV = (rows - 1) * stride + ks virtual rows starting at input row
// y0 * stride - pad, WP = W + 2 * pad columns starting at input column -pad.  A tap of an output pixel is then always
// inside the staged block, so phase B needs no bounds checks.
__device__ __forceinline__ int strip_virtual_rows(const PackParams & p, int y0, int y1) { return (y1 - y0 - 1) * p.stride + p.ks; }

// Phase B of the word path: assembles the packed rows of output rows y0..y1-1 for the channel blocks cb0..cb0+cbn-1
// (group g) from the staged block.  A thread owns one uint4 (4 K-words) position of the group's range and walks the
// strip's pixels with it: the four offsets into the staged block are worked out once, and per pixel there remain four
// shared loads, one 16-byte store and a few additions -- no table, no division, no bounds check.  `lanes` threads share a
// pixel (all of the group's uint4 positions when there are at most PK_THREADS of them), so consecutive threads write
// consecutive 16-byte pieces of one row and then of the next.
template <bool WIN>
__device__ __forceinline__ void words_phase_b_impl(const PackParams & p, const uint32_t * s_words, int b, int g, int y0, int y1,
		int RV, int WP, int CB, int cb0, int cbn)
{
	const int taps = p.ks * p.ks;
	const int new_k = CB * taps;
	const bool last_group = (g == p.groups - 1);
	const int q_lo = (cb0 * taps) >> 2;                                   // cb0 % 4 == 0 whenever groups > 1
	const int q_hi = last_group ? (p.ldw >> 2) : (((cb0 + cbn) * taps) >> 2);
	const int nq = q_hi - q_lo;
	const int lanes = min(nq, PK_THREADS);
	const uint32_t m_lanes = last_group ? p.m_nq[1] : p.m_nq[0];
	const int slots = fast_div(PK_THREADS, lanes, m_lanes);               // pixels worked on at the same time
	const int slot = fast_div(threadIdx.x, lanes, m_lanes);
	const int lane = threadIdx.x - slot * lanes;
	if (slot >= slots) { return; }                                        // PK_THREADS % lanes left-over threads
	const int pixels = (y1 - y0) * p.OW;
	const int yl0 = fast_div(slot, p.OW, p.m_ow), x0 = slot - yl0 * p.OW;
	const int d_yl = fast_div(slots, p.OW, p.m_ow), d_x = slots - d_yl * p.OW;
	const int d_base = (d_yl * WP + d_x) * p.stride;                      // staged offset of a pixel: (yl * WP + x) * stride
	const int wrap_base = (WP - p.OW) * p.stride;                         // extra when x runs over the end of an output row
	const int ldq = p.ldw >> 2;
	uint4 * const out_img = reinterpret_cast<uint4 *>(p.out) + (size_t)b * p.OH * p.OW * ldq;
	for (int wq = lane; wq < nq; wq += lanes)
	{
		int e[4];
		#pragma unroll
		for (int u = 0; u < 4; ++u)
		{
			const int wi = (q_lo + wq) * 4 + u;
			const int cb = fast_div(wi, taps, p.m_taps);
			const int t = wi - cb * taps;
			const int ky = fast_div(t, p.ks, p.m_ks);
			e[u] = (wi < new_k) ? ((cb - cb0) * RV + ky) * WP + (t - ky * p.ks) : -1;      // -1: padding word of the row
		}
		int yl = yl0, x = x0;
		int base = (yl0 * WP + x0) * p.stride;
		uint4 * dst = out_img + (size_t)(y0 * p.OW + slot) * ldq + q_lo + wq;               // row-major rows: a constant step per round
		const size_t d_dst = (size_t)slots * ldq;
		for (int pl = slot; pl < pixels; pl += slots)
		{
			uint4 v;
			v.x = (e[0] >= 0) ? s_words[base + e[0]] : 0u;
			v.y = (e[1] >= 0) ? s_words[base + e[1]] : 0u;
			v.z = (e[2] >= 0) ? s_words[base + e[2]] : 0u;
			v.w = (e[3] >= 0) ? s_words[base + e[3]] : 0u;
			if (WIN)
			{
				const int oy = y0 + yl;
				out_img[(size_t)(((oy >> 1) * p.win_w + (x >> 1)) * 4 + (oy & 1) * 2 + (x & 1)) * ldq + q_lo + wq] = v;
				yl += d_yl;
			}
			else
			{
				*dst = v;
				dst += d_dst;
			}
			x += d_x; base += d_base;
			if (x >= p.OW) { x -= p.OW; base += wrap_base; if (WIN) { ++yl; } }
		}
	}
}

__device__ __forceinline__ void words_phase_b(const PackParams & p, const uint32_t * s_words, int b, int g, int y0, int y1,
		int RV, int WP, int CB, int cb0, int cbn)
{
	if (p.win_w > 0) { words_phase_b_impl<true>(p, s_words, b, g, y0, y1, RV, WP, CB, cb0, cbn); }
	else { words_phase_b_impl<false>(p, s_words, b, g, y0, y1, RV, WP, CB, cb0, cbn); }
}

// ---- word path -----------------------------------------------------------------------------
// shared: packed[cb_local][R][W] words, R = input rows of this strip.
// VEC  = floats per load (4, 2 or 1, as the row pitch and pointer alignment allow);
// SUBS = threads sharing one output word, each covering 32/SUBS channels (4 on small problems, to put more threads
//        to work; 1 on large ones, where a thread then keeps 32 independent loads in flight).
// POOL = the tensor in memory is max-pooled on the fly (always with VEC == 1: pooled pixels are not contiguous).
template <int VEC, int SUBS, bool POOL = false>
__global__ void __launch_bounds__(PK_THREADS, 4)
pack_input_words_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int rest = fast_div((int)blockIdx.x, p.groups, p.m_groups);
	const int g = (int)blockIdx.x - rest * p.groups;
	const int b = fast_div(rest, p.tiles_per_image, p.m_tiles);
	const int tile = rest - b * p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int iy_v0 = y0 * p.stride - p.pad;  // input row of staged row 0 (may be negative: padding)
	const int iy_lo = max(iy_v0, 0);
	const int iy_hi = min((y1 - 1) * p.stride - p.pad + p.ks - 1, p.H - 1);
	const int R = iy_hi - iy_lo + 1;          // rows that exist in the image; may be <= 0 when the strip only sees padding
	const int RV = strip_virtual_rows(p, y0, y1);
	const int WP = p.W + 2 * p.pad;
	const int CB = p.C >> 5;
	const int cb0 = g * p.cb_per_cta;
	const int cbn = min(p.cb_per_cta, CB - cb0);
	const int span = max(R, 0) * p.W;         // contiguous floats per channel
	const size_t chan_stride = POOL ? (size_t)p.in_h * p.in_w : (size_t)p.H * p.W;
	const float * img = p.in + ((size_t)b * p.C + (size_t)cb0 * 32) * chan_stride + (POOL ? 0 : (size_t)iy_lo * p.W);

	// the padding around the rows phase A fills
	if (p.pad > 0 || R < RV)
	{
		for (int i = threadIdx.x; i < cbn * RV * WP; i += PK_THREADS) { s_words[i] = 0u; }
		__syncthreads();
	}
	const int stage0 = (iy_lo - iy_v0) * WP + p.pad;   // staged offset of image element (iy_lo, 0)

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
			if (POOL)
			{
				// ev = (staged row, column) of the pooled tensor; src - ev is element 0 of the first unpooled plane
				const int rl = ev / p.W;
				const int xl = ev - rl * p.W;
				#pragma unroll
				for (int ch = 0; ch < CH; ++ch)
				{
					w[0] |= (pooled_positive(src - ev + (size_t)ch * chan_stride, p, iy_lo + rl, xl) ? 1u : 0u) << ch;
				}
			}
			else
			{
				// Loads are issued in explicit batches (all loads of a batch before the first compare) so that a thread
				// keeps LB independent requests in flight; the kernel is bound by memory latency otherwise.
				constexpr int LB = (CH < 16) ? CH : 16;
				#pragma unroll
				for (int ch0 = 0; ch0 < CH; ch0 += LB)
				{
					float v[LB][VEC];
					#pragma unroll
					for (int u = 0; u < LB; ++u)
					{
						const float * q = src + (size_t)(ch0 + u) * chan_stride;
						if (VEC == 4)
						{
							const float4 t = __ldg(reinterpret_cast<const float4 *>(q));
							v[u][0] = t.x; v[u][1 % VEC] = t.y; v[u][2 % VEC] = t.z; v[u][3 % VEC] = t.w;
						}
						else if (VEC == 2)
						{
							const float2 t = __ldg(reinterpret_cast<const float2 *>(q));
							v[u][0] = t.x; v[u][1 % VEC] = t.y;
						}
						else
						{
							v[u][0] = __ldg(q);
						}
					}
					#pragma unroll
					for (int u = 0; u < LB; ++u)
					{
						#pragma unroll
						for (int j = 0; j < VEC; ++j) { w[j] |= (v[u][j] > 0 ? 1u : 0u) << (ch0 + u); }
					}
				}
			}
			// VEC divides W, so the VEC positions share a row
			const int r = (ev * VEC) / p.W;
			const int at = (cbl * RV + r) * WP + stage0 + (ev * VEC - r * p.W);
			if (SUBS == 1)
			{
				#pragma unroll
				for (int j = 0; j < VEC; ++j) { s_words[at + j] = w[j]; }
			}
			else
			{
				// SUBS == 4: this thread owns byte `sub` of each word
				uint8_t * dst = reinterpret_cast<uint8_t *>(s_words + at) + sub;
				#pragma unroll
				for (int j = 0; j < VEC; ++j) { dst[j * 4] = (uint8_t)w[j]; }
			}
		}
	}
	__syncthreads();

	words_phase_b(p, s_words, b, g, y0, y1, RV, WP, CB, cb0, cbn);
}

// The same packing when the previous xnor layer already left its output as sign bits, 32 channels per word
// ([image][C/32][in_h*in_w], written by the sign-only GEMM epilogue): phase A is a copy of words -- or, with a
// max-pool in between, the OR of the window's words, because sign(max) is the OR of the signs.  The fp32
// activation tensor and the pooled tensor are never written.
__global__ void __launch_bounds__(PK_THREADS)
pack_input_from_signs_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int rest = fast_div((int)blockIdx.x, p.groups, p.m_groups);
	const int g = (int)blockIdx.x - rest * p.groups;
	const int b = fast_div(rest, p.tiles_per_image, p.m_tiles);
	const int tile = rest - b * p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int iy_v0 = y0 * p.stride - p.pad;
	const int RV = strip_virtual_rows(p, y0, y1);
	const int WP = p.W + 2 * p.pad;
	const int CB = p.C >> 5;
	const int cb0 = g * p.cb_per_cta;
	const int cbn = min(p.cb_per_cta, CB - cb0);
	const size_t plane = (size_t)p.in_h * p.in_w;
	const uint32_t * bits = reinterpret_cast<const uint32_t *>(p.in) + ((size_t)b * CB + cb0) * plane;
	// phase A walks the staged block itself, padding included: a warp takes four staged rows at a time (four independent
	// loads per lane), lanes run along the row
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	constexpr int NW = PK_THREADS / 32;
	const uint32_t m_rv = p.m_rv[(y1 - y0 == p.rows_per_cta) ? 0 : 1];
	const int units = cbn * RV;
	for (int u0 = warp; u0 < units; u0 += 4 * NW)
	{
		const uint32_t * src[4];
		bool ok[4];
		#pragma unroll
		for (int k = 0; k < 4; ++k)
		{
			const int u = min(u0 + k * NW, units - 1);
			const int cbl = fast_div(u, RV, m_rv);
			const int iy = iy_v0 + (u - cbl * RV);
			ok[k] = (u0 + k * NW < units) && iy >= 0 && iy < p.H;
			src[k] = bits + (size_t)cbl * plane;
			if (p.pool_size == 0) { src[k] += (ptrdiff_t)iy * p.W - p.pad; }
			else { src[k] += (ptrdiff_t)(iy * p.pool_stride - p.pool_off) * p.in_w; }      // first window row
		}
		for (int cv = lane; cv < WP; cv += 32)
		{
			const int ix = cv - p.pad;
			const bool col_ok = (ix >= 0 && ix < p.W);
			uint32_t v[4];
			#pragma unroll
			for (int k = 0; k < 4; ++k)
			{
				uint32_t word = 0;
				if (ok[k] && col_ok)
				{
					if (p.pool_size == 0)
					{
						word = __ldg(src[k] + cv);
					}
					else
					{
						// src[k] is row py0 of the unpooled plane; rows and columns outside the image are skipped
						const int u = u0 + k * NW;
						const int iy = iy_v0 + (u - fast_div(u, RV, m_rv) * RV);
						const int py0 = iy * p.pool_stride - p.pool_off;
						const int px0 = ix * p.pool_stride - p.pool_off;
						if (p.pool_size == 2)
						{
							// the usual window: four independent loads
							const bool r0 = (py0 >= 0 && py0 < p.in_h), r1 = (py0 + 1 >= 0 && py0 + 1 < p.in_h);
							const bool c0 = (px0 >= 0 && px0 < p.in_w), c1 = (px0 + 1 >= 0 && px0 + 1 < p.in_w);
							const uint32_t * q = src[k] + px0;
							const uint32_t a = (r0 && c0) ? __ldg(q) : 0u;
							const uint32_t b2 = (r0 && c1) ? __ldg(q + 1) : 0u;
							const uint32_t c2 = (r1 && c0) ? __ldg(q + p.in_w) : 0u;
							const uint32_t d2 = (r1 && c1) ? __ldg(q + p.in_w + 1) : 0u;
							word = (a | b2) | (c2 | d2);
						}
						else
						for (int l = 0; l < p.pool_size; ++l)
						{
							if (py0 + l < 0 || py0 + l >= p.in_h) { continue; }
							for (int m = 0; m < p.pool_size; ++m)
							{
								const int xx = px0 + m;
								if (xx >= 0 && xx < p.in_w) { word |= __ldg(src[k] + (ptrdiff_t)l * p.in_w + xx); }
							}
						}
					}
				}
				v[k] = word;
			}
			#pragma unroll
			for (int k = 0; k < 4; ++k)
			{
				const int u = u0 + k * NW;
				if (u < units) { s_words[u * WP + cv] = v[k]; }
			}
		}
	}
	__syncthreads();
	words_phase_b(p, s_words, b, g, y0, y1, RV, WP, CB, cb0, cbn);
}

// Phase A of the bit kernels: planes[c][rr][xw] = ballot of (input(c, iy0 + rr, 32*xw + lane - pad) > 0).
// One warp walks whole plane rows, eight words (eight independent loads per lane) at a time; the only integer
// division is one per plane row.
__device__ __forceinline__ void build_bit_planes(const float * img, size_t chan_stride, const PackParams & p,
		int RR, int PW, int iy0)
{
	extern __shared__ uint32_t s_words[];
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	constexpr int NWARPS = PK_THREADS / 32;
	constexpr int UNROLL = 8;
	if (p.from_planes)
	{
		// the producer already made x-packed sign words; a staged word is two of them shifted by the padding
		const int GW = (p.W + 31) >> 5;
		const uint32_t * planes = reinterpret_cast<const uint32_t *>(img);
		for (int cr = warp; cr < p.C * RR; cr += NWARPS)
		{
			const int c = cr / RR;
			const int rr = cr - c * RR;
			const int iy = iy0 + rr;
			const bool row_ok = (iy >= 0 && iy < p.H);
			const uint32_t * g = planes + ((size_t)c * p.H + (row_ok ? iy : 0)) * GW;
			for (int xw = lane; xw < PW; xw += 32)
			{
				const int first = 32 * xw - p.pad;               // image column of bit 0 of this staged word
				const int w0 = first >> 5;
				const uint32_t lo = (row_ok && w0 >= 0 && w0 < GW) ? __ldg(g + w0) : 0u;
				const uint32_t hi = (row_ok && w0 + 1 >= 0 && w0 + 1 < GW) ? __ldg(g + w0 + 1) : 0u;
				s_words[(size_t)cr * PW + xw] = __funnelshift_r(lo, hi, first & 31);
			}
		}
		return;
	}
	for (int cr = warp; cr < p.C * RR; cr += NWARPS)
	{
		const int c = cr / RR;
		const int rr = cr - c * RR;
		const int iy = iy0 + rr;
		const bool row_ok = (iy >= 0 && iy < p.H);
		const float * row = img + (size_t)c * chan_stride + (size_t)iy * p.W - p.pad + lane;
		uint32_t * dst = s_words + (size_t)cr * PW;
		for (int xw0 = 0; xw0 < PW; xw0 += UNROLL)
		{
			float v[UNROLL];
			#pragma unroll
			for (int u = 0; u < UNROLL; ++u)
			{
				const int ix = (xw0 + u) * 32 + lane - p.pad;
				const bool ok = row_ok && xw0 + u < PW && ix >= 0 && ix < p.W;
				if (p.pool_size > 0)
				{
					v[u] = (ok && pooled_positive(img + (size_t)c * chan_stride, p, iy, ix)) ? 1.0f : 0.0f;
				}
				else
				{
					v[u] = ok ? __ldg(row + (xw0 + u) * 32) : 0.0f;
				}
			}
			#pragma unroll
			for (int u = 0; u < UNROLL; ++u)
			{
				const uint32_t word = __ballot_sync(0xffffffffu, v[u] > 0);
				if (lane == 0 && xw0 + u < PW) { dst[xw0 + u] = word; }
			}
		}
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
	const size_t chan_stride = (p.pool_size > 0) ? (size_t)p.in_h * p.in_w : (size_t)p.H * p.W;
	const float * img = p.from_planes ? p.in + (size_t)b * p.C * p.H * ((p.W + 31) >> 5)       // 4-byte words either way
	                                  : p.in + (size_t)b * p.C * chan_stride;
	const int iy0 = y0 * p.stride - p.pad;

	// phase A: one warp ballot per 32 consecutive padded positions of one (channel, row)
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	build_bit_planes(img, chan_stride, p, RR, PW, iy0);
	__syncthreads();

	// phase B: thread builds 4 consecutive K-words (bits k0 .. k0+127) of one output row.
	// K order: k = (c*ks + ky)*ks + kx, i.e. consecutive groups (c, ky) of ks bits each.
	const int ldq = p.ldw >> 2;
	const int pixels = (y1 - y0) * p.OW;
	const int n_groups = p.C * p.ks;
	const uint32_t tap_mask = (p.ks >= 32) ? 0xffffffffu : ((1u << p.ks) - 1u);
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
		reinterpret_cast<uint4 *>(p.out + out_row(p, b, y0 + yl, x) * p.ldw)[wq] = make_uint4(v[0], v[1], v[2], v[3]);
	}
}

// Stride-1 bit path.  Same bit planes as above; phase B works on 32x32 bit blocks held in registers:
// a thread gathers, for 32 consecutive K indices, the 32-pixel words "tap (c, ky, kx) of pixels x0 .. x0+31"
// (one funnel shift each, because with stride 1 those taps are adjacent plane bits), transposes the block with
// five butterfly stages, and stores one K-word for each of the 32 pixels.  That is about 0.8 instructions per
// output bit instead of a dozen, which is what lets the small-channel layers approach memory speed.
__device__ __forceinline__ void transpose32(uint32_t (&A)[32])
{
	// out[l] bit k == in[k] bit l  (bit 0 = least significant)
	uint32_t m = 0x0000ffffu;
	#pragma unroll
	for (int j = 16; j != 0; j >>= 1)
	{
		#pragma unroll
		for (int k = 0; k < 32; k = (k + j + 1) & ~j)
		{
			const uint32_t t = ((A[k] >> j) ^ A[k + j]) & m;
			A[k + j] ^= t;
			A[k] ^= t << j;
		}
		m ^= m << (j >> 1);
	}
}

__global__ void __launch_bounds__(PK_THREADS)
pack_input_bits_s1_kernel(const PackParams p)
{
	extern __shared__ uint32_t s_words[];
	const int tile = blockIdx.x % p.tiles_per_image;
	const int b = blockIdx.x / p.tiles_per_image;
	const int y0 = tile * p.rows_per_cta;
	const int y1 = min(y0 + p.rows_per_cta, p.OH);
	const int RR = (y1 - y0 - 1) + p.ks;
	const int PW = ((p.W + 2 * p.pad + 31) >> 5) + 1;
	const size_t chan_stride = (p.pool_size > 0) ? (size_t)p.in_h * p.in_w : (size_t)p.H * p.W;
	const float * img = p.from_planes ? p.in + (size_t)b * p.C * p.H * ((p.W + 31) >> 5)       // 4-byte words either way
	                                  : p.in + (size_t)b * p.C * chan_stride;
	const int iy0 = y0 - p.pad;

	// phase A: one warp ballot per 32 consecutive padded positions of one (channel, row)
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	build_bit_planes(img, chan_stride, p, RR, PW, iy0);
	__syncthreads();

	// phase B: task = (output row yl, 32-pixel chunk pc, K-word kb); consecutive threads take consecutive kb
	const int chunks = (p.OW + 31) >> 5;
	const int tasks = (y1 - y0) * chunks * p.ldw;
	const int taps = p.ks * p.ks;
	for (int t = threadIdx.x; t < tasks; t += PK_THREADS)
	{
		const int kb = t % p.ldw;
		const int rest = t / p.ldw;
		const int pc = rest % chunks;
		const int yl = rest / chunks;
		const int x0 = pc * 32;
		uint32_t * dst = p.out + kb;
		const bool win = (p.win_w > 0);
		const size_t r0 = out_row(p, b, y0 + yl, x0);      // x0 is a multiple of 32: the 32 pixels are 16 window halves in a row
		const int npix = min(32, p.OW - x0);
		int k = kb * 32;
		if (k >= p.K)
		{
			for (int l = 0; l < npix; ++l) { dst[(r0 + (win ? (size_t)((l >> 1) * 4 + (l & 1)) : (size_t)l)) * p.ldw] = 0u; }
			continue;
		}
		int c = k / taps;
		int tt = k - c * taps;
		int ky = tt / p.ks;
		int kx = tt - ky * p.ks;
		const uint32_t * plane = s_words + ((size_t)c * RR + yl + ky) * PW + pc;
		uint32_t A[32];
		#pragma unroll
		for (int kk = 0; kk < 32; ++kk)
		{
			A[kk] = (k < p.K) ? __funnelshift_r(plane[0], plane[1], kx) : 0u;
			++k;
			if (++kx == p.ks)
			{
				kx = 0;
				plane += PW;
				if (++ky == p.ks) { ky = 0; plane += (size_t)(RR - p.ks) * PW; }
			}
		}
		transpose32(A);
		#pragma unroll
		for (int l = 0; l < 32; ++l)
		{
			if (l < npix) { dst[(r0 + (win ? (size_t)((l >> 1) * 4 + (l & 1)) : (size_t)l)) * p.ldw] = A[l]; }
		}
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


// ---- first pass of the two-pass word path -------------------------------------------------------
// input [blocks][32][hw] fp32 -> words [blocks][hw], bit ch of a word = input(block, ch, e) > 0; `blocks` = images x
// 32-channel blocks.  A pure stream: a thread owns VEC consecutive positions of one block and keeps 16 independent
// VEC-wide loads in flight, twice; no shared memory, no halo, nothing read twice.
// Loads written as volatile inline PTX: the compiler otherwise folds load, compare and OR into a chain with a handful of
// loads in flight, and this kernel lives on bytes in flight.
template <int VEC> struct StreamLoad;
template <> struct StreamLoad<4>
{
	static __device__ __forceinline__ void ld(const float * p, float (&v)[4])
	{
		asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "l"(p));
	}
};
template <> struct StreamLoad<2>
{
	static __device__ __forceinline__ void ld(const float * p, float (&v)[2])
	{
		asm volatile("ld.global.nc.L1::no_allocate.v2.f32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "l"(p));
	}
};
template <> struct StreamLoad<1>
{
	static __device__ __forceinline__ void ld(const float * p, float (&v)[1])
	{
		asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v[0]) : "l"(p));
	}
};

template <int VEC>
__global__ void __launch_bounds__(PK_THREADS)
sign_words_kernel(const float * __restrict__ in, uint32_t * __restrict__ words, int hwv, long long items)
{
	const long long idx = (long long)blockIdx.x * PK_THREADS + threadIdx.x;
	if (idx >= items) { return; }
	const long long blk = idx / hwv;
	const int ev = (int)(idx - blk * hwv);
	const size_t hw = (size_t)hwv * VEC;
	const float * src = in + (size_t)blk * 32 * hw + (size_t)ev * VEC;
	uint32_t w[VEC];
	#pragma unroll
	for (int j = 0; j < VEC; ++j) { w[j] = 0; }
	#pragma unroll
	for (int ch0 = 0; ch0 < 32; ch0 += 16)
	{
		float v[16][VEC];
		#pragma unroll
		for (int u = 0; u < 16; ++u) { StreamLoad<VEC>::ld(src + (size_t)(ch0 + u) * hw, v[u]); }
		#pragma unroll
		for (int u = 0; u < 16; ++u)
		{
			#pragma unroll
			for (int j = 0; j < VEC; ++j) { w[j] |= (v[u][j] > 0 ? 1u : 0u) << (ch0 + u); }
		}
	}
	uint32_t * dst = words + (size_t)blk * hw + (size_t)ev * VEC;
	if (VEC == 4) { *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1 % VEC], w[2 % VEC], w[3 % VEC]); }
	else if (VEC == 2) { *reinterpret_cast<uint2 *>(dst) = make_uint2(w[0], w[1 % VEC]); }
	else { dst[0] = w[0]; }
}

size_t pack_words_bytes(const xnor_b200_conv_desc & d)
{
	if (d.c % 32 != 0) { return 0; }
	return round_up((size_t)d.batch * (d.c / 32) * d.h * d.w * 4, 256);
}

static int launch_sign_words(const xnor_b200_conv_desc & d, const float * input, uint32_t * words, cudaStream_t stream)
{
	const size_t hw = (size_t)d.h * d.w;
	const long long blocks = (long long)d.batch * (d.c / 32);
	const bool a16 = (((uintptr_t)input | (uintptr_t)words) & 15u) == 0;
	const bool a8 = (((uintptr_t)input | (uintptr_t)words) & 7u) == 0;
	// the widest loads that still give every SM a CTA: bytes in flight per thread are what the kernel lives on
	const long long min_items = (long long)sm_count() * PK_THREADS;
	int vec = 1;
	if (hw % 4 == 0 && a16 && blocks * (long long)(hw / 4) >= min_items) { vec = 4; }
	else if (hw % 2 == 0 && a8 && blocks * (long long)(hw / 2) >= min_items) { vec = 2; }
	const long long items = blocks * (long long)(hw / vec);
	const long long grid = (items + PK_THREADS - 1) / PK_THREADS;
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	if (vec == 4) { sign_words_kernel<4><<<(unsigned)grid, PK_THREADS, 0, stream>>>(input, words, (int)(hw / 4), items); }
	else if (vec == 2) { sign_words_kernel<2><<<(unsigned)grid, PK_THREADS, 0, stream>>>(input, words, (int)(hw / 2), items); }
	else { sign_words_kernel<1><<<(unsigned)grid, PK_THREADS, 0, stream>>>(input, words, (int)hw, items); }
	return check_launch();
}

int launch_pack_input(const xnor_b200_conv_desc & d, const xnor_b200_pool_desc * pool, const float * input,
		uint32_t * t_bit_input, cudaStream_t stream, int from_signs, int window_major, uint32_t * words_scratch)
{
	// Two passes on request: a streaming pass leaves the sign words, the staging kernel then reads those (1/32 of the
	// bytes, out of L2) instead of the floats.  Measured against the single kernel it only draws level on the largest maps.
	if (words_scratch != nullptr && !from_signs && pool == nullptr && d.c % 32 == 0 && tuning().pack_two_pass == 2)
	{
		const int rc = launch_sign_words(d, input, words_scratch, stream);
		if (rc != XNOR_B200_OK) { return rc; }
		return launch_pack_input(d, nullptr, reinterpret_cast<const float *>(words_scratch), t_bit_input, stream, 1, window_major, nullptr);
	}
	if (from_signs && d.c % 32 != 0 && pool != nullptr) { return XNOR_B200_ERR_INVALID; }     // sign planes are made at the size the convolution sees
	PackParams p;
	p.from_planes = (from_signs && d.c % 32 != 0) ? 1 : 0;
	p.win_w = 0;
	p.pool_size = 0; p.pool_stride = 1; p.pool_off = 0; p.in_h = d.h; p.in_w = d.w; p.pool_fast = 0;
	if (pool != nullptr)
	{
		if (pool->size <= 0 || pool->stride <= 0 || pool->pad < 0 || pool->in_h <= 0 || pool->in_w <= 0) { return XNOR_B200_ERR_INVALID; }
		// the convolution must be described on the pooled tensor (src-lib/maxpool_layer.cpp:129-130)
		if (d.h != (pool->in_h + pool->pad - pool->size) / pool->stride + 1
				|| d.w != (pool->in_w + pool->pad - pool->size) / pool->stride + 1) { return XNOR_B200_ERR_INVALID; }
		p.pool_size = pool->size; p.pool_stride = pool->stride; p.pool_off = pool->pad / 2;
		p.in_h = pool->in_h; p.in_w = pool->in_w;
		p.pool_fast = (pool->size == 2 && pool->stride == 2 && pool->pad / 2 == 0 && pool->in_h % 2 == 0 && pool->in_w % 2 == 0
				&& (((uintptr_t)input) & 7u) == 0) ? 1 : 0;
	}
	p.in = input;
	p.out = t_bit_input;
	p.C = d.c; p.H = d.h; p.W = d.w;
	p.OH = conv_out_dim(d.h, d.size, d.stride, d.pad);
	p.OW = conv_out_dim(d.w, d.size, d.stride, d.pad);
	if (window_major)
	{
		if (p.OH % 2 != 0 || p.OW % 2 != 0) { return XNOR_B200_ERR_INVALID; }
		p.win_w = p.OW / 2;
	}
	p.ks = d.size; p.stride = d.stride; p.pad = d.pad;
	p.K = d.size * d.size * d.c;
	p.ldw = aligned_lda(p.K) / 32;
	const bool word_path = (d.c % 32 == 0);
	if (d.size > 63) { return XNOR_B200_ERR_TOO_LARGE; }             // kernel offsets are kept in 6-bit fields
	// CTAs to aim for.  Each CTA loads, synchronises, then stores, so overlap of loads and stores comes from
	// several CTAs sharing an SM.  xnor_b200_set_tuning may override the factor.
	const int ctas_per_sm = (tuning().pack_ctas_per_sm > 0) ? tuning().pack_ctas_per_sm : 4;
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
		const size_t row_bytes = (size_t)cb_per_cta * (d.w + 2 * d.pad) * 4;       // one staged row, padding columns included
		if (row_bytes * (size_t)in_rows(1) > PK_MAX_SMEM) { return XNOR_B200_ERR_TOO_LARGE; }
		// rounded down: a grid a little over what fits at once costs a second, nearly empty wave
		const int strips = (int)min((long long)p.OH, max(1LL, want_ctas / ctas));
		int rows = (p.OH + strips - 1) / strips;
		const size_t room = PK_MAX_SMEM;
		while (rows > 1 && row_bytes * (size_t)in_rows(rows) > room) { --rows; }
		p.rows_per_cta = rows;
		p.tiles_per_image = (p.OH + rows - 1) / rows;
		const size_t words_bytes = round_up(row_bytes * (size_t)in_rows(rows), 16);
		{
			const int taps = d.size * d.size, wp = d.w + 2 * d.pad;
			const int nq_first = (cb_per_cta * taps) >> 2;
			const int nq_last = (p.ldw >> 2) - (((p.groups - 1) * cb_per_cta * taps) >> 2);
			const int last_rows = p.OH - (p.tiles_per_image - 1) * rows;
			p.m_groups = div_magic(p.groups); p.m_tiles = div_magic(p.tiles_per_image);
			p.m_ow = div_magic(p.OW); p.m_wp = div_magic(wp); p.m_taps = div_magic(taps); p.m_ks = div_magic(d.size);
			p.m_nq[0] = div_magic(min(nq_first, PK_THREADS)); p.m_nq[1] = div_magic(min(nq_last, PK_THREADS));
			p.m_rv[0] = div_magic(in_rows(rows)); p.m_rv[1] = div_magic(in_rows(last_rows));
		}
		const size_t smem = words_bytes;
		const long long grid = (long long)d.batch * p.tiles_per_image * p.groups;
		if (grid > 0x7fffffffLL || grid * max(p.groups, p.tiles_per_image) > 0xffffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }   // fast_div range
		const int vec = (pool != nullptr) ? 1
				: ((d.w % 4 == 0) && (((uintptr_t)input & 15u) == 0)) ? 4
				: ((d.w % 2 == 0) && (((uintptr_t)input & 7u) == 0)) ? 2 : 1;
		// words per CTA in phase A; below two per thread the channel split keeps more threads busy
		const long long words_per_cta = (long long)cb_per_cta * min(in_rows(rows), d.h) * d.w;
		const bool split = words_per_cta < (long long)PK_THREADS * vec;
		void (*kern)(const PackParams) =
				vec == 4 ? (split ? pack_input_words_kernel<4, 4> : pack_input_words_kernel<4, 1>)
				: vec == 2 ? (split ? pack_input_words_kernel<2, 4> : pack_input_words_kernel<2, 1>)
				: (pool != nullptr) ? (split ? pack_input_words_kernel<1, 4, true> : pack_input_words_kernel<1, 1, true>)
				: (split ? pack_input_words_kernel<1, 4> : pack_input_words_kernel<1, 1>);
		if (from_signs) { kern = pack_input_from_signs_kernel; }
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
		// Phase A of the bit kernels is a chain of dependent load rounds per warp, so short strips (many CTAs in
		// flight) hide its latency better than long ones; 8 rows keep the halo re-reads at (size-1)/8.
		rows = min(rows, 8);
		p.rows_per_cta = rows;
		p.tiles_per_image = (p.OH + rows - 1) / rows;
		const size_t smem = round_up(row_bytes * (size_t)in_rows(rows), 16);
		const long long grid = (long long)d.batch * p.tiles_per_image;
		if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
		void (*kern)(const PackParams) = (d.stride == 1) ? pack_input_bits_s1_kernel : pack_input_bits_kernel;
		int rc = ensure_dynamic_smem((const void *)kern, smem > 48 * 1024 ? PK_MAX_SMEM : 0);
		if (rc != XNOR_B200_OK) { return rc; }
		kern<<<(unsigned)grid, PK_THREADS, smem, stream>>>(p);
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
	return launch_pack_input(*desc, nullptr, input, (uint32_t *)t_bit_input, (cudaStream_t)stream);
}

extern "C" size_t xnor_b200_pack_words_bytes(const xnor_b200_conv_desc * desc)
{
	if (desc == nullptr || validate_desc(desc) != XNOR_B200_OK) { return 0; }
	return pack_words_bytes(*desc);
}

extern "C" int xnor_b200_pack_input_staged(const xnor_b200_conv_desc * desc, const float * input, uint32_t * words,
		uint8_t * t_bit_input, void * stream)
{
	if (desc == nullptr || input == nullptr || words == nullptr || t_bit_input == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (desc->c % 32 != 0) { return XNOR_B200_ERR_INVALID; }
	if (((uintptr_t)t_bit_input & 15u) != 0 || ((uintptr_t)words & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	return launch_pack_input(*desc, nullptr, input, (uint32_t *)t_bit_input, (cudaStream_t)stream, 0, 0, words);
}

extern "C" int xnor_b200_pack_input_pooled(const xnor_b200_conv_desc * desc, const xnor_b200_pool_desc * pool,
		const float * input, uint8_t * t_bit_input, void * stream)
{
	if (desc == nullptr || pool == nullptr || input == nullptr || t_bit_input == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (((uintptr_t)t_bit_input & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	return launch_pack_input(*desc, pool, input, (uint32_t *)t_bit_input, (cudaStream_t)stream);
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
