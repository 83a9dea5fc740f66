// XNOR-popcount GEMM with the per-filter mean scale, bias, leaky/linear activation and optional
// shortcut add fused into the epilogue.
//
// Replaces gemm_nn_custom_bin_mean_transposed_gpu (src-lib/im2col_kernels.cu:793-956, :1156-1193; a wmma
// b1 kernel that reads both operands straight from global memory, one warp per 8x16 outputs) and, on the
// CPU side, gemm_nn_custom_bin_mean_transposed + add_bias + leaky (src-lib/gemm.cpp:907-1019,
// src-lib/convolutional_layer.cpp:1269-1289, src-lib/gemm.cpp:1472-1498).
//
// Operands: A [M][lda_words] and B [n_total][ldb_words] 32-bit words, K bits of data per row followed by
// zero bits.  With zero padding on both sides  popc(a ^ b)  over whole words counts exactly the
// disagreeing bits among the first K, so   2*count - K  =  K - 2*sum popc(a ^ b)   with no padding
// correction term (the reference subtracts f1 because its A padding is complemented).
//
// Tiling: a CTA computes a BM x BN tile over one K slice; operands are staged through a STAGES-deep cp.async
// ring in shared memory (row pitch KT+4 words so that 16-byte reads of 8 consecutive rows hit 32 distinct
// banks); every thread owns a TM x TN register tile of int32 accumulators and consumes four K-words per
// 16-byte shared load.
//
// Split-K over a thread-block cluster: layers with many filters but few output pixels (13x13 maps at batch 1)
// have too few tiles to occupy 148 SMs.  For those the K range is divided among the S CTAs of a (1,1,S)
// cluster; the non-leading CTAs park their integer partial sums in their own shared memory, and the leading
// CTA adds them through distributed shared memory before running the epilogue.  No global scratch, no
// atomics, no second launch, and the sums stay exact integers in any order.
//
// The epilogue mirrors the reference CPU rounding order: one fp32 multiply, one fp32 add, then the leaky blend
// -- never a fused multiply-add.
#include "xnor_common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace xnor
{

struct GemmParams
{
	const uint32_t * A;
	const uint32_t * B;
	int M, n_total, n_per_image, K;
	int lda_words, ldb_words;
	int kw;                 // K-words to visit in total, multiple of 4 (<= lda_words, ldb_words)
	int kw_slice;           // K-words per cluster rank, multiple of 4
	int split;              // cluster size along K (gridDim.z)
	float * C;
	int ldc;
	const float * mean_arr;
	const float * bias;
	int leaky;
	const float * shortcut_in;
	float * shortcut_out;
	int32_t * counts;       // when set: write integer agreement counts [M][n_total] instead of C
	uint32_t * signs;       // when set: write only the sign bits of the output, 32 filters per word: [img][M/32][pixel]
	int tiles_m, tiles_n;
	GemmExtra x;            // window-major column order and direct sign sinks (all zero: none)
};

__device__ __forceinline__ void cp_async_16(uint32_t * smem_dst, const uint32_t * gmem_src, bool valid)
{
	const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
	const int src_bytes = valid ? 16 : 0;   // 0 -> the 16 destination bytes are zero-filled
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

template <int BM, int BN, int TM, int TN, int KT, int STAGES>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
xnor_gemm_kernel(const GemmParams p)
{
	constexpr int TX = BN / TN;
	constexpr int TY = BM / TM;
	constexpr int NT = TX * TY;
	constexpr int PITCH = KT + 4;               // words
	constexpr int A_STAGE = BM * PITCH;
	constexpr int B_STAGE = BN * PITCH;
	constexpr int CHUNKS_ROW = KT / 4;          // 16-byte chunks per staged row
	static_assert(KT % 4 == 0, "KT must be a multiple of 4 words");
	static_assert(STAGES * (BM + BN) * PITCH >= NT * TM * TN, "ring too small to park split-K partial sums");

	extern __shared__ __align__(16) uint32_t smem[];
	uint32_t * sA = smem;
	uint32_t * sB = smem + STAGES * A_STAGE;

	// Tiles that share a B tile are adjacent in launch order, so concurrently running CTAs re-use the
	// same packed-activation rows out of L2 while A (small) stays resident.
	const int tile_m = blockIdx.x % p.tiles_m;
	const int tile_n = blockIdx.x / p.tiles_m;
	const int m0 = tile_m * BM;
	const int n0 = tile_n * BN;
	const int tx = threadIdx.x % TX;
	const int ty = threadIdx.x / TX;
	const int k_begin = blockIdx.z * p.kw_slice;
	const int k_end = min(k_begin + p.kw_slice, p.kw);

	auto load_stage = [&](int stage, int k0)
	{
		uint32_t * dA = sA + stage * A_STAGE;
		uint32_t * dB = sB + stage * B_STAGE;
		for (int ch = threadIdx.x; ch < BM * CHUNKS_ROW; ch += NT)
		{
			const int r = ch / CHUNKS_ROW;
			const int kc = (ch - r * CHUNKS_ROW) * 4;
			if (k0 + kc >= k_end) { continue; }          // never read by the compute loop
			const bool ok = (m0 + r < p.M);
			const uint32_t * src = ok ? p.A + (size_t)(m0 + r) * p.lda_words + k0 + kc : p.A;
			cp_async_16(dA + r * PITCH + kc, src, ok);
		}
		for (int ch = threadIdx.x; ch < BN * CHUNKS_ROW; ch += NT)
		{
			const int r = ch / CHUNKS_ROW;
			const int kc = (ch - r * CHUNKS_ROW) * 4;
			if (k0 + kc >= k_end) { continue; }
			const bool ok = (n0 + r < p.n_total);
			const uint32_t * src = ok ? p.B + (size_t)(n0 + r) * p.ldb_words + k0 + kc : p.B;
			cp_async_16(dB + r * PITCH + kc, src, ok);
		}
	};

	int acc[TM][TN];
	#pragma unroll
	for (int i = 0; i < TM; ++i)
	{
		#pragma unroll
		for (int j = 0; j < TN; ++j) { acc[i][j] = 0; }
	}

	const int num_kt = (max(k_end - k_begin, 0) + KT - 1) / KT;
	#pragma unroll
	for (int s = 0; s < STAGES - 1; ++s)
	{
		if (s < num_kt) { load_stage(s, k_begin + s * KT); }
		cp_async_commit();
	}

	for (int kt = 0; kt < num_kt; ++kt)
	{
		cp_async_wait<STAGES - 2>();
		__syncthreads();
		{
			const int nk = kt + STAGES - 1;
			if (nk < num_kt) { load_stage(nk % STAGES, k_begin + nk * KT); }
			cp_async_commit();
		}
		const uint32_t * cA = sA + (kt % STAGES) * A_STAGE + ty * PITCH;
		const uint32_t * cB = sB + (kt % STAGES) * B_STAGE + tx * PITCH;
		auto step = [&](int k4)
		{
			uint4 a[TM], b[TN];
			#pragma unroll
			for (int i = 0; i < TM; ++i) { a[i] = *reinterpret_cast<const uint4 *>(cA + i * TY * PITCH + k4); }
			#pragma unroll
			for (int j = 0; j < TN; ++j) { b[j] = *reinterpret_cast<const uint4 *>(cB + j * TX * PITCH + k4); }
			#pragma unroll
			for (int i = 0; i < TM; ++i)
			{
				#pragma unroll
				for (int j = 0; j < TN; ++j)
				{
					acc[i][j] += __popc(a[i].x ^ b[j].x) + __popc(a[i].y ^ b[j].y)
							+ __popc(a[i].z ^ b[j].z) + __popc(a[i].w ^ b[j].w);
				}
			}
		};
		const int kvalid = min(KT, k_end - k_begin - kt * KT);   // the last stage of a slice may hold fewer words
		if (kvalid == KT)
		{
			#pragma unroll
			for (int k4 = 0; k4 < KT; k4 += 4) { step(k4); }
		}
		else
		{
			for (int k4 = 0; k4 < kvalid; k4 += 4) { step(k4); }
		}
	}
	cp_async_wait<0>();

	// Split-K: fold the partial sums of cluster ranks 1..S-1 into rank 0 through distributed shared memory.
	if (p.split > 1)
	{
		cg::cluster_group cluster = cg::this_cluster();
		__syncthreads();                                   // everyone is done reading the operand ring
		int * park = reinterpret_cast<int *>(smem);        // [TM*TN][NT]: consecutive threads, consecutive words
		if (blockIdx.z != 0)
		{
			#pragma unroll
			for (int i = 0; i < TM; ++i)
			{
				#pragma unroll
				for (int j = 0; j < TN; ++j) { park[(i * TN + j) * NT + threadIdx.x] = acc[i][j]; }
			}
		}
		cluster.sync();
		if (blockIdx.z == 0)
		{
			for (int r = 1; r < p.split; ++r)
			{
				const int * peer = cluster.map_shared_rank(park, r);
				#pragma unroll
				for (int i = 0; i < TM; ++i)
				{
					#pragma unroll
					for (int j = 0; j < TN; ++j) { acc[i][j] += peer[(i * TN + j) * NT + threadIdx.x]; }
				}
			}
		}
		cluster.sync();                                    // peers keep their shared memory alive until it has been read
		if (blockIdx.z != 0) { return; }
	}

	// Sign-only epilogue: the next layer binarises this output anyway, so only (value > 0) is kept, packed 32
	// filters to a word in the channel-packed layout the next pack kernel stages in shared memory.  Bytes go
	// through shared memory because one thread's register tile holds filters that are TY rows apart.
	if (p.signs != nullptr || p.x.n_sinks > 0)
	{
		constexpr int SP = BN + 4;
		static_assert(BM % 32 == 0 && BN % 4 == 0 && BM * SP + (BM / 32) * BN * 4 <= STAGES * (BM + BN) * PITCH * 4, "sign staging does not fit the ring");
		uint8_t * s_sign = reinterpret_cast<uint8_t *>(smem);
		__syncthreads();                                   // the operand ring (or the parked sums) is dead from here on
		#pragma unroll
		for (int i = 0; i < TM; ++i)
		{
			const int ml = i * TY + ty;
			const int m = m0 + ml;
			const float mean = (m < p.M) ? __ldg(p.mean_arr + m) : 0.0f;
			const float bias = (m < p.M && p.bias != nullptr) ? __ldg(p.bias + m) : 0.0f;
			#pragma unroll
			for (int j = 0; j < TN; ++j)
			{
				float v = __fmul_rn((float)(p.K - 2 * acc[i][j]), mean);
				if (p.bias != nullptr) { v = __fadd_rn(v, bias); }
				s_sign[ml * SP + j * TX + tx] = (m < p.M && v > 0.0f) ? 1 : 0;
			}
		}
		__syncthreads();
		// one thread per (32-filter word, column): assemble the word, keep it in shared memory for the sinks
		const int mwords = p.M >> 5;
		uint32_t * s_wd = smem + (BM * SP) / 4;                                  // [(BM/32)][BN], behind the sign bytes
		for (int idx = threadIdx.x; idx < (BM / 32) * BN; idx += NT)
		{
			const int wl = idx / BN;
			const int cl = idx - wl * BN;
			uint32_t word = 0;
			#pragma unroll
			for (int k = 0; k < 32; ++k) { word |= (uint32_t)s_sign[(wl * 32 + k) * SP + cl] << k; }
			s_wd[idx] = word;
			const int col = n0 + cl;
			const int mw = (m0 >> 5) + wl;
			if (p.signs != nullptr && col < p.n_total && mw < mwords)
			{
				const int img = col / p.n_per_image;
				p.signs[((size_t)img * mwords + mw) * p.n_per_image + col_to_pixel(p.x, col - img * p.n_per_image)] = word;
			}
		}
		if (p.x.n_sinks > 0) { __syncthreads(); }
		// sinks: one task per (word, column or window, copy, tap), spread over the whole CTA
		#pragma unroll
		for (int si = 0; si < 2; ++si)
		{
			if (si >= p.x.n_sinks) { break; }
			const SinkParams & s = p.x.sinks[si];
			const int cols = (s.pool != 0) ? BN / 4 : BN;
			const int copies = (s.up == 2) ? 4 : 1;
			const int tasks = (BM / 32) * cols * copies * s.taps;
			for (int t = threadIdx.x; t < tasks; t += NT)
			{
				int r = t;
				const int cg_ = r % cols;  r /= cols;
				const int tap = r % s.taps; r /= s.taps;
				const int cp = r % copies;
				const int wl = r / copies;
				const int mw = (m0 >> 5) + wl;
				if (mw >= mwords) { continue; }
				if (s.pool != 0)
				{
					const int col = n0 + cg_ * 4;
					if (col >= p.n_total) { continue; }
					const uint4 w4 = *reinterpret_cast<const uint4 *>(s_wd + wl * BN + cg_ * 4);
					const int img = col / p.n_per_image;
					const int q = (col - img * p.n_per_image) >> 2;      // window index: the four columns are one 2x2 window
					const int wy = q / p.x.win_w;
					sink_store_tap(s, img, wy, q - wy * p.x.win_w, mw, tap, w4.x | w4.y | w4.z | w4.w);
				}
				else
				{
					const int col = n0 + cg_;
					if (col >= p.n_total) { continue; }
					const int img = col / p.n_per_image;
					const int pix = col_to_pixel(p.x, col - img * p.n_per_image);
					int oy = pix / p.x.out_w;
					int ox = pix - oy * p.x.out_w;
					if (s.up == 2) { oy = 2 * oy + (cp >> 1); ox = 2 * ox + (cp & 1); }
					sink_store_tap(s, img, oy, ox, mw, tap, s_wd[wl * BN + cg_]);
				}
			}
		}
		if (p.C == nullptr) { return; }
	}

	// epilogue
	// The shortcut operand of all TM x TN outputs is requested first: one load per output in program order (each
	// behind the previous output's stores) would cost a thread a full memory latency per output.
	float sc[TM][TN];
	if (p.shortcut_out != nullptr)
	{
		#pragma unroll
		for (int j = 0; j < TN; ++j)
		{
			const int col = n0 + j * TX + tx;
			const int img = col / p.n_per_image;
			const int pix = col_to_pixel(p.x, col - img * p.n_per_image);
			#pragma unroll
			for (int i = 0; i < TM; ++i)
			{
				const int m = m0 + i * TY + ty;
				sc[i][j] = (col < p.n_total && m < p.M) ? __ldcs(p.shortcut_in + ((size_t)img * p.M + m) * p.ldc + pix) : 0.0f;
			}
		}
	}
	#pragma unroll
	for (int j = 0; j < TN; ++j)
	{
		const int col = n0 + j * TX + tx;
		if (col >= p.n_total) { continue; }
		const int img = col / p.n_per_image;
		const int pix = col_to_pixel(p.x, col - img * p.n_per_image);
		#pragma unroll
		for (int i = 0; i < TM; ++i)
		{
			const int m = m0 + i * TY + ty;
			if (m >= p.M) { continue; }
			if (p.counts != nullptr)
			{
				p.counts[(size_t)m * p.n_total + col] = p.K - acc[i][j];
				continue;
			}
			const size_t idx = ((size_t)img * p.M + m) * p.ldc + pix;
			const float dot = (float)(p.K - 2 * acc[i][j]);
			float v = __fmul_rn(dot, __ldg(p.mean_arr + m));
			if (p.bias != nullptr) { v = __fadd_rn(v, __ldg(p.bias + m)); }
			if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
			if (p.C != nullptr) { p.C[idx] = v; }
			if (p.shortcut_out != nullptr) { p.shortcut_out[idx] = __fadd_rn(sc[i][j], v); }
		}
	}
}

// ---- short-K kernel ---------------------------------------------------------------------------
// Layers with very short rows (K <= 256 bits: 16 channels x 3x3, or a 1x1 layer over <= 256 channels) on a small batch.  The tiled kernel above
// spends ~110 instructions per output on them (ring management, staging, per-output index arithmetic) for ~15 that
// are arithmetic.  Here a thread keeps the packed row of ONE pixel in registers and walks the 32 filters of its
// filter group, whose packed rows sit in shared memory and are read as broadcasts: per (pixel, filter) KW4 16-byte
// loads, 4*KW4 XOR + POPC + ADD, one multiply-add for the value.  The thread ends up holding the complete sign word of
// its pixel, so the sign outputs and sinks need no staging: a pooled sink is an OR over the four lanes of a window.
constexpr int SK_THREADS = 128;

// FPT = filters per thread (32: a thread owns the whole sign word of its pixel; 8: four neighbouring lanes share a
// pixel and combine their byte of the word with two shuffles -- used when there are too few pixels to fill the GPU).
// TAIL = K words that carry data in the last 16-byte group (1..4): the words behind them are zero in both operands
// and are not visited (a 16-channel 3x3 layer has 4.5 data words in its 8-word row).
template <int KW4, int FPT, int TAIL>
__global__ void __launch_bounds__(SK_THREADS)
xnor_gemm_smallk_kernel(const GemmParams p)
{
	constexpr int SUBS = 32 / FPT;
	__shared__ __align__(16) uint32_t s_a[32 * KW4 * 4];
	__shared__ float2 s_mb[32];                               // (mean, bias) of the group's filters
	const int m0 = blockIdx.y * 32;
	if (threadIdx.x < 32)
	{
		const int m = m0 + threadIdx.x;
		s_mb[threadIdx.x] = make_float2((m < p.M) ? __ldg(p.mean_arr + m) : 0.0f, (m < p.M && p.bias != nullptr) ? __ldg(p.bias + m) : 0.0f);
	}
	for (int i = threadIdx.x; i < 32 * KW4; i += SK_THREADS)
	{
		const int f = i / KW4;
		const int q = i - f * KW4;
		uint4 v = make_uint4(0u, 0u, 0u, 0u);
		if (m0 + f < p.M) { v = __ldg(reinterpret_cast<const uint4 *>(p.A + (size_t)(m0 + f) * p.lda_words) + q); }
		reinterpret_cast<uint4 *>(s_a)[i] = v;
	}
	const int sub = threadIdx.x % SUBS;
	const int col = blockIdx.x * (SK_THREADS / SUBS) + threadIdx.x / SUBS;
	const bool live = (col < p.n_total);
	const int img = live ? col / p.n_per_image : 0;
	const int pixcol = live ? col - img * p.n_per_image : 0;
	const int pix = col_to_pixel(p.x, pixcol);
	uint4 b[KW4];
	if (KW4 <= 2 && p.x.masks != nullptr)
	{
		// Tap-major rows: bits [t*C, t*C + C) are the channel mask of the pixel under tap t (zero outside the image).
		// C is 8 or 16, so a mask never straddles a word.
		uint32_t w[KW4 * 4];
		#pragma unroll
		for (int i = 0; i < KW4 * 4; ++i) { w[i] = 0u; }
		const int y = pix / p.x.pl_w;
		const int x = pix - y * p.x.pl_w;
		const int C = p.x.pl_c;
		const uint8_t * img_masks = p.x.masks + (size_t)img * p.x.pl_h * p.x.pl_w * (C >> 3);
		#pragma unroll
		for (int t = 0; t < 9; ++t)
		{
			const int iy = y + t / 3 - 1;
			const int ix = x + t % 3 - 1;
			uint32_t m = 0u;
			if (live && iy >= 0 && iy < p.x.pl_h && ix >= 0 && ix < p.x.pl_w)
			{
				const size_t e = (size_t)iy * p.x.pl_w + ix;
				m = (C == 16) ? (uint32_t)__ldg(reinterpret_cast<const uint16_t *>(img_masks) + e) : (uint32_t)__ldg(img_masks + e);
			}
			// bit offset t*C: compile-time for each of the two channel counts
			if (C == 16) { if (t * 16 < KW4 * 128) { w[(t * 16) >> 5] |= m << ((t * 16) & 31); } }
			else         { if (t * 8 < KW4 * 128) { w[(t * 8) >> 5] |= m << ((t * 8) & 31); } }
		}
		#pragma unroll
		for (int q = 0; q < KW4; ++q) { b[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]); }
	}
	else if (FPT == 8 && KW4 <= 2 && p.x.planes != nullptr)
	{
		// The packed row of this pixel straight from the sign planes: bits (c*3 + ky)*3 + kx = plane c, row y + ky - 1,
		// columns x - 1 .. x + 1 (zero outside the image; bits behind the last column are zero in the planes).  The four
		// lanes of a pixel split the work by kernel row: lane ky gathers its 3 bits of every channel at bit c*9, shifts
		// the whole row left by 3*ky, and an OR across the four lanes (lane 3 adds nothing) gives everyone the full row.
		uint32_t w[KW4 * 4 + 1];
		#pragma unroll
		for (int i = 0; i < KW4 * 4 + 1; ++i) { w[i] = 0u; }
		const int y = pix / p.x.pl_w;
		const int x = pix - y * p.x.pl_w;
		const int gw = (p.x.pl_w + 31) >> 5;
		const int w0 = (x - 1) >> 5;                       // -1 for x == 0: that word reads as zero
		const int sh = (x - 1) & 31;
		const int iy = y + sub - 1;
		const bool row_ok = live && sub < 3 && iy >= 0 && iy < p.x.pl_h;
		const uint32_t * rows = p.x.planes + ((size_t)img * p.x.pl_c * p.x.pl_h + (row_ok ? iy : 0)) * gw;
		#pragma unroll
		for (int c = 0; c < KW4 * 128 / 9; ++c)
		{
			if (c < p.x.pl_c && row_ok)
			{
				const uint32_t * row = rows + (size_t)c * p.x.pl_h * gw;
				const uint32_t lo = (w0 >= 0) ? __ldg(row + w0) : 0u;
				const uint32_t hi = (w0 + 1 < gw) ? __ldg(row + w0 + 1) : 0u;
				const uint32_t bits = __funnelshift_r(lo, hi, sh) & 7u;
				const int o = c * 9;                           // compile-time after unrolling
				w[o >> 5] |= bits << (o & 31);
				if ((o & 31) > 29) { w[(o >> 5) + 1] |= bits >> (32 - (o & 31)); }
			}
		}
		const int lsh = 3 * sub;                               // 0, 3, 6 (9 for the idle lane, whose words are zero)
		#pragma unroll
		for (int i = KW4 * 4; i > 0; --i) { w[i] = __funnelshift_l(w[i - 1], w[i], lsh); }
		w[0] <<= lsh;
		#pragma unroll
		for (int i = 0; i < KW4 * 4; ++i)
		{
			w[i] |= __shfl_xor_sync(0xffffffffu, w[i], 1);
			w[i] |= __shfl_xor_sync(0xffffffffu, w[i], 2);
		}
		#pragma unroll
		for (int q = 0; q < KW4; ++q) { b[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]); }
	}
	else
	{
		#pragma unroll
		for (int q = 0; q < KW4; ++q)
		{
			b[q] = live ? __ldg(reinterpret_cast<const uint4 *>(p.B + (size_t)col * p.ldb_words) + q) : make_uint4(0u, 0u, 0u, 0u);
		}
	}
	__syncthreads();

	uint32_t word = 0;
	#pragma unroll 4
	for (int ff = 0; ff < FPT; ++ff)
	{
		const int f = sub * FPT + ff;
		const int m = m0 + f;
		if (m >= p.M) { break; }
		int cnt = 0;
		#pragma unroll
		for (int q = 0; q < KW4; ++q)
		{
			const uint4 a = reinterpret_cast<const uint4 *>(s_a)[f * KW4 + q];
			cnt += __popc(a.x ^ b[q].x);
			if (q < KW4 - 1 || TAIL > 1) { cnt += __popc(a.y ^ b[q].y); }
			if (q < KW4 - 1 || TAIL > 2) { cnt += __popc(a.z ^ b[q].z); }
			if (q < KW4 - 1 || TAIL > 3) { cnt += __popc(a.w ^ b[q].w); }
		}
		const float2 mb = s_mb[f];
		float v = __fmul_rn((float)(p.K - 2 * cnt), mb.x);
		if (p.bias != nullptr) { v = __fadd_rn(v, mb.y); }
		word |= (v > 0.0f ? 1u : 0u) << f;
		if (p.C != nullptr && live)
		{
			if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
			p.C[((size_t)img * p.M + m) * p.ldc + pix] = v;
		}
	}
	if (p.signs == nullptr && p.x.n_sinks == 0) { return; }
	#pragma unroll
	for (int o = 1; o < SUBS; o <<= 1) { word |= __shfl_xor_sync(0xffffffffu, word, o); }
	const int mwords = p.M >> 5;
	const int mw = blockIdx.y;
	if (p.signs != nullptr && live && sub == 0) { p.signs[((size_t)img * mwords + mw) * p.n_per_image + pix] = word; }
	#pragma unroll
	for (int si = 0; si < 2; ++si)
	{
		if (si >= p.x.n_sinks) { break; }
		const SinkParams & s = p.x.sinks[si];
		if (s.pool != 0)
		{
			// window-major columns: the lanes of columns 4w .. 4w+3 hold one 2x2 window and share the taps of its pooled word
			uint32_t w = live ? word : 0u;
			w |= __shfl_xor_sync(0xffffffffu, w, SUBS);
			w |= __shfl_xor_sync(0xffffffffu, w, 2 * SUBS);
			if (!live) { continue; }
			const int q = pixcol >> 2;
			const int wy = q / p.x.win_w;
			const int wx = q - wy * p.x.win_w;
			for (int tap = (col & 3) * SUBS + sub; tap < s.taps; tap += 4 * SUBS) { sink_store_tap(s, img, wy, wx, mw, tap, w); }
		}
		else if (live)
		{
			const int oy = pix / p.x.out_w;
			const int ox = pix - oy * p.x.out_w;
			const int copies = (s.up == 2) ? 4 : 1;
			for (int t = sub; t < copies * s.taps; t += SUBS)
			{
				const int cp = t / s.taps;
				const int tap = t - cp * s.taps;
				const int iy = (s.up == 2) ? 2 * oy + (cp >> 1) : oy;
				const int ix = (s.up == 2) ? 2 * ox + (cp & 1) : ox;
				sink_store_tap(s, img, iy, ix, mw, tap, word);
			}
		}
	}
}

template <int KW4, int TAIL>
static int launch_smallk(const GemmParams & p, cudaStream_t stream)
{
	const int gy = (p.M + 31) / 32;
	// enough pixels to give every SM a few hundred threads: one pixel per thread, else four lanes per pixel
	const bool wide = ((long long)p.n_total * gy >= (long long)sm_count() * 256) && p.x.planes == nullptr;   // rows from planes: built in the four-lane variant
	const int cols_per_cta = wide ? SK_THREADS : SK_THREADS / 4;
	const long long gx = ((long long)p.n_total + cols_per_cta - 1) / cols_per_cta;
	if (gx > 0x7fffffffLL || gy > 65535) { return XNOR_B200_ERR_TOO_LARGE; }
	if (wide) { xnor_gemm_smallk_kernel<KW4, 32, TAIL><<<dim3((unsigned)gx, (unsigned)gy, 1), SK_THREADS, 0, stream>>>(p); }
	else { xnor_gemm_smallk_kernel<KW4, 8, TAIL><<<dim3((unsigned)gx, (unsigned)gy, 1), SK_THREADS, 0, stream>>>(p); }
	return check_launch();
}

// ---- one-shot kernel ---------------------------------------------------------------------------
// Mid-sized layers on a small batch (13x13 and 26x26 maps with hundreds of filters and K up to a few thousand bits):
// the ring, the cluster and its barriers in the tiled kernel cost more than the arithmetic.  Here a CTA owns 32 filters x
// 32 pixels and loads everything it needs once: the 32 filter rows into shared memory, and every thread its own slice of
// its pixel's row straight into registers.  The 8 warps split K (warp w takes the w-th slice of KS4 16-byte groups);
// lane = pixel; a thread walks the 32 filters with broadcast reads, exactly like the short-K kernel.  The eight partial
// counts per output are added through shared memory (integers: exact in any order), then warp w finishes filters
// 4w .. 4w+3 of its lane's pixel and warp 0 assembles the sign word for the sign outputs and sinks.
constexpr int OS_THREADS = 256;
constexpr int OS_WARPS = OS_THREADS / 32;

// FT = filters per CTA: 32, or 16 for layers that only write fp32 (no sign word to assemble) and whose 32-filter tiles would
// leave the GPU with one and a bit waves.
template <int KS4, int FT>
__global__ void __launch_bounds__(OS_THREADS)
xnor_gemm_oneshot_kernel(const GemmParams p)
{
	constexpr int SLICE = KS4 * 4;                 // K words per warp
	constexpr int KWP = OS_WARPS * SLICE;          // K words per (zero-padded) row in shared memory
	extern __shared__ __align__(16) uint32_t smem[];
	constexpr int FPW = FT / OS_WARPS;             // filters a warp finishes
	uint32_t * s_a = smem;                                             // [FT][KWP]
	int * s_red = reinterpret_cast<int *>(smem + FT * KWP);            // [8 warps][FT filters][32 pixels]
	uint8_t * s_bits = reinterpret_cast<uint8_t *>(smem + FT * KWP + OS_WARPS * FT * 32);   // [8 warps][32 pixels]
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	const int m0 = blockIdx.y * FT;
	const int col = blockIdx.x * 32 + lane;
	const bool live = (col < p.n_total);

	for (int i = threadIdx.x; i < FT * (KWP / 4); i += OS_THREADS)
	{
		const int f = i / (KWP / 4);
		const int q = i - f * (KWP / 4);
		uint4 v = make_uint4(0u, 0u, 0u, 0u);
		if (m0 + f < p.M && q * 4 < p.kw) { v = __ldg(reinterpret_cast<const uint4 *>(p.A + (size_t)(m0 + f) * p.lda_words) + q); }
		reinterpret_cast<uint4 *>(s_a)[i] = v;
	}
	uint4 b[KS4];
	#pragma unroll
	for (int q = 0; q < KS4; ++q)
	{
		const int w4 = warp * KS4 + q;                 // 16-byte group of the row
		b[q] = (live && w4 * 4 < p.kw) ? __ldg(reinterpret_cast<const uint4 *>(p.B + (size_t)col * p.ldb_words) + w4) : make_uint4(0u, 0u, 0u, 0u);
	}
	__syncthreads();

	#pragma unroll 4
	for (int f = 0; f < FT; ++f)
	{
		const uint4 * ar = reinterpret_cast<const uint4 *>(s_a + f * KWP + warp * SLICE);
		int cnt = 0;
		#pragma unroll
		for (int q = 0; q < KS4; ++q)
		{
			const uint4 a = ar[q];
			cnt += __popc(a.x ^ b[q].x) + __popc(a.y ^ b[q].y) + __popc(a.z ^ b[q].z) + __popc(a.w ^ b[q].w);
		}
		s_red[(warp * FT + f) * 32 + lane] = cnt;
	}
	__syncthreads();

	const int img = live ? col / p.n_per_image : 0;
	const int pixcol = live ? col - img * p.n_per_image : 0;
	const int pix = col_to_pixel(p.x, pixcol);
	uint32_t bits = 0;
	#pragma unroll
	for (int ff = 0; ff < FPW; ++ff)
	{
		const int f = warp * FPW + ff;
		const int m = m0 + f;
		int cnt = 0;
		#pragma unroll
		for (int w = 0; w < OS_WARPS; ++w) { cnt += s_red[(w * FT + f) * 32 + lane]; }
		if (m < p.M)
		{
			float v = __fmul_rn((float)(p.K - 2 * cnt), __ldg(p.mean_arr + m));
			if (p.bias != nullptr) { v = __fadd_rn(v, __ldg(p.bias + m)); }
			bits |= (v > 0.0f ? 1u : 0u) << ff;
			if (p.C != nullptr && live)
			{
				if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
				p.C[((size_t)img * p.M + m) * p.ldc + pix] = v;
			}
		}
	}
	if (p.signs == nullptr && p.x.n_sinks == 0) { return; }
	s_bits[warp * 32 + lane] = (uint8_t)bits;
	__syncthreads();
	// the CTA's FT sign bits of this lane's pixel: the whole 32-filter word, or one 16-bit half of it.  Every warp assembles
	// it; warp 0 stores the sign words, the sink taps are dealt out over the 8 warps.
	uint32_t word = 0;
	#pragma unroll
	for (int w = 0; w < OS_WARPS; ++w) { word |= (uint32_t)s_bits[w * 32 + lane] << (FPW * w); }
	const int mwords = p.M >> 5;
	const int mw = (FT == 32) ? blockIdx.y : blockIdx.y >> 1;
	const int half = (FT == 32) ? -1 : (blockIdx.y & 1);
	if (p.signs != nullptr && live && warp == 0)
	{
		uint32_t * dst = p.signs + ((size_t)img * mwords + mw) * p.n_per_image + pix;
		if (half < 0) { *dst = word; }
		else { reinterpret_cast<uint16_t *>(dst)[half] = (uint16_t)word; }
	}
	#pragma unroll
	for (int si = 0; si < 2; ++si)
	{
		if (si >= p.x.n_sinks) { break; }
		const SinkParams & s = p.x.sinks[si];
		if (s.pool != 0)
		{
			// window-major columns: lanes 4w .. 4w+3 hold one 2x2 window; its taps go to (warp, lane of the window) pairs
			uint32_t w = live ? word : 0u;
			w |= __shfl_xor_sync(0xffffffffu, w, 1);
			w |= __shfl_xor_sync(0xffffffffu, w, 2);
			if (!live) { continue; }
			const int q = pixcol >> 2;
			const int wy = q / p.x.win_w;
			const int wx = q - wy * p.x.win_w;
			for (int tap = warp * 4 + (col & 3); tap < s.taps; tap += 4 * OS_WARPS) { sink_store_tap(s, img, wy, wx, mw, tap, w, half); }
		}
		else if (live)
		{
			const int oy = pix / p.x.out_w;
			const int ox = pix - oy * p.x.out_w;
			const int copies = (s.up == 2) ? 4 : 1;
			for (int t = warp; t < copies * s.taps; t += OS_WARPS)
			{
				const int cp = t / s.taps;
				const int tap = t - cp * s.taps;
				sink_store_tap(s, img, (s.up == 2) ? 2 * oy + (cp >> 1) : oy, (s.up == 2) ? 2 * ox + (cp & 1) : ox, mw, tap, word, half);
			}
		}
	}
}

template <int KS4, int FT>
static int launch_oneshot(const GemmParams & p, cudaStream_t stream)
{
	const long long gx = ((long long)p.n_total + 31) / 32;
	const int gy = (p.M + FT - 1) / FT;
	if (gx > 0x7fffffffLL || gy > 65535) { return XNOR_B200_ERR_TOO_LARGE; }
	const size_t smem = (size_t)(FT * OS_WARPS * KS4 * 4 + OS_WARPS * FT * 32) * 4 + OS_WARPS * 32;
	int rc = ensure_dynamic_smem((const void *)xnor_gemm_oneshot_kernel<KS4, FT>, smem);
	if (rc != XNOR_B200_OK) { return rc; }
	xnor_gemm_oneshot_kernel<KS4, FT><<<dim3((unsigned)gx, (unsigned)gy, 1), OS_THREADS, smem, stream>>>(p);
	return check_launch();
}

// Problems whose 32x32 output tiles fit the GPU in a single wave, with rows of at most 8 x 32 words.  Measured on B200:
// 512x169x2304 7.0 vs 8.6 us, 256x169x1024 4.0 vs 5.0 us against the tiled kernel; with more tiles than SMs (1024x169x4608:
// 192 tiles) the busiest SM gets two CTAs of POPC work and the tiled kernel with cluster split-K wins (13.8 vs 16.1 us).
// Returns the filter tile to use (32 or 16), 0 when the tiled kernel should keep the layer.  16-filter tiles (a CTA then owns
// one 16-bit half of every sign word): layers with a bit more than one wave of 32-filter tiles (256x676x3456: 176 tiles ->
// 352 half tiles, 10.1 vs 12.9 us; 1024x169x4608: 12.2 vs 14.1 us).
static int oneshot_problem(int M, int n_total, int kw, bool fp32_only)
{
	(void)fp32_only;
	if (kw <= 8 || kw > OS_WARPS * 32 || tuning().gemm_route >= XNOR_B200_ROUTE_TENSOR) { return 0; }
	const long long ntiles = ((long long)n_total + 31) / 32;
	if ((long long)((M + 31) / 32) * ntiles <= (long long)sm_count()) { return 32; }
	if (M % 32 == 0 && (long long)((M + 15) / 16) * ntiles <= 3ll * sm_count() && (long long)((M + 31) / 32) * ntiles <= 2ll * sm_count()) { return 16; }
	return 0;
}

// ---- configurations ----------------------------------------------------------------------------

struct TileConfig
{
	int bm, bn;
	int warps;              // warps per CTA
	int max_resident;       // CTAs that fit on one SM (threads / shared memory)
	float store_cost;       // epilogue cycles per output (narrow thread columns coalesce worse)
	int (*launch)(GemmParams &, cudaStream_t);
};

template <int BM, int BN, int TM, int TN, int KT, int STAGES>
static int launch_config(GemmParams & p, cudaStream_t stream)
{
	constexpr int NT = (BM / TM) * (BN / TN);
	constexpr size_t SMEM = (size_t)STAGES * (BM + BN) * (KT + 4) * 4;
	auto kern = xnor_gemm_kernel<BM, BN, TM, TN, KT, STAGES>;
	int rc = ensure_dynamic_smem((const void *)kern, SMEM);
	if (rc != XNOR_B200_OK) { return rc; }
	p.tiles_m = (p.M + BM - 1) / BM;
	p.tiles_n = (p.n_total + BN - 1) / BN;
	const long long grid = (long long)p.tiles_m * p.tiles_n;
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }

	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3((unsigned)grid, 1, (unsigned)p.split);
	cfg.blockDim = dim3(NT, 1, 1);
	cfg.dynamicSmemBytes = SMEM;
	cfg.stream = stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = 1;
	attr[0].val.clusterDim.y = 1;
	attr[0].val.clusterDim.z = (unsigned)p.split;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
	if (e != cudaSuccess) { return cuda_fail(e); }
	return check_launch();
}

// Measured on B200: the POPC unit is the limiter for every register tile and it only saturates with about 20
// resident warps per SM, so small tiles with many co-resident CTAs (index 2..5) beat the classic large tiles
// (0, 1: one 8-warp CTA per SM, latency-bound); the large ones are kept for the tuning sweep only.
static const TileConfig g_configs[] = {
	{128, 128, 8,  1, 0.30f, launch_config<128, 128, 8, 8, 32, 3>},
	{ 64, 128, 8,  2, 0.30f, launch_config< 64, 128, 4, 8, 32, 3>},
	{ 64,  64, 8,  4, 0.30f, launch_config< 64,  64, 4, 4, 32, 3>},
	{ 32, 128, 8,  6, 0.25f, launch_config< 32, 128, 4, 4, 16, 3>},
	{ 32,  64, 8,  8, 0.30f, launch_config< 32,  64, 2, 4, 16, 3>},
	{ 32,  32, 4, 14, 0.60f, launch_config< 32,  32, 2, 4, 16, 3>},
};
constexpr int NUM_CONFIGS = (int)(sizeof(g_configs) / sizeof(g_configs[0]));

// Estimated duration in SM cycles of one launch.  CTAs on one SM share its POPC unit (one warp instruction every
// other cycle per SM when enough warps are resident), so the busiest SM sets the time; stores add a per-output
// cost; every launch pays a fixed latency for its first loads, and a cluster pays for the reduction.
static float estimate_cycles(const TileConfig & c, int M, int n_total, int kw, int split, int sms)
{
	const long long tiles = (long long)((M + c.bm - 1) / c.bm) * ((n_total + c.bn - 1) / c.bn) * split;
	const long long per_sm = (tiles + sms - 1) / sms;
	const int kw_slice = (int)round_up((size_t)(kw + split - 1) / split, 4);
	const float resident_warps = (float)min(per_sm, (long long)c.max_resident) * c.warps;
	const float eff = fminf(1.0f, 0.3f + resident_warps / 30.0f);
	const float cta_cycles = (float)c.bm * c.bn / 32.0f * kw_slice * 2.0f / eff;
	const float store_cycles = (float)c.bm * c.bn * c.store_cost / split;
	const float fixed = 4000.0f + (split > 1 ? 3000.0f + 200.0f * split : 0.0f);
	return per_sm * (cta_cycles + store_cycles) + 700.0f * ((per_sm + c.max_resident - 1) / c.max_resident) + fixed;
}

// rows_in_kernel: the kernel would build its rows from planes / masks, i.e. the alternative is a pack kernel plus a GEMM
// over a 32-byte-per-pixel operand; that pays at every size, the plain short-K kernel only while launches dominate.
static bool short_k_problem(int M, int n_total, int kw, bool rows_in_kernel = false)
{
	return kw <= 8 && (rows_in_kernel || (long long)M * n_total <= (4ll << 20)) && tuning().gemm_route < XNOR_B200_ROUTE_TENSOR;
}

bool gemm_takes_planes(int M, int n_total, int c, int size, int stride, int pad)
{
	const int K = c * size * size;
	return size == 3 && stride == 1 && pad == 1 && c % 32 != 0 && K <= 256
			&& short_k_problem(M, n_total, (int)round_up((size_t)(K + 31) / 32, 4), true);
}

int launch_xnor_gemm(int M, int n_total, int n_per_image, int K,
		const uint32_t * A, int lda_words, const uint32_t * B, int ldb_words,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky,
		const float * shortcut_in, float * shortcut_out, int32_t * counts, cudaStream_t stream, uint32_t * signs,
		const GemmExtra * extra)
{
	const bool sum_signs = (extra != nullptr && (extra->sum_signs != nullptr || extra->sum_rows != nullptr));
	// signs of the fused shortcut sum: written by the tensor-core kernel's fp32 epilogue only
	if (sum_signs && (shortcut_out == nullptr || M % 32 != 0 || counts != nullptr || signs != nullptr || extra->n_sinks > 0)) { return XNOR_B200_ERR_INVALID; }
	const bool extras = (extra != nullptr && (extra->win_w > 0 || extra->n_sinks > 0 || extra->planes != nullptr || extra->masks != nullptr || sum_signs));
	if ((signs != nullptr || (extra != nullptr && extra->n_sinks > 0)) && M % 32 != 0) { return XNOR_B200_ERR_INVALID; }
	if (extras && counts != nullptr) { return XNOR_B200_ERR_INVALID; }
	if (extras && n_per_image % 4 != 0 && (extra->win_w > 0)) { return XNOR_B200_ERR_INVALID; }
	if (extras)
	{
		if (extra->n_sinks < 0 || extra->n_sinks > 2) { return XNOR_B200_ERR_INVALID; }
		for (int i = 0; i < extra->n_sinks; ++i)
		{
			if (extra->sinks[i].pool != 0 && extra->win_w <= 0) { return XNOR_B200_ERR_INVALID; }   // a window must be four consecutive columns
		}
	}
	GemmParams p;
	p.x = GemmExtra();
	if (extra != nullptr) { p.x = *extra; }
	if (p.x.out_w <= 0) { p.x.out_w = 1; }
	p.signs = signs;
	p.A = A; p.B = B;
	p.M = M; p.n_total = n_total; p.n_per_image = n_per_image; p.K = K;
	p.lda_words = lda_words; p.ldb_words = ldb_words;
	p.kw = (int)round_up((size_t)(K + 31) / 32, 4);
	p.C = C; p.ldc = ldc; p.mean_arr = mean_arr; p.bias = bias; p.leaky = leaky;
	p.shortcut_in = shortcut_in; p.shortcut_out = shortcut_out; p.counts = counts;

	// Large layers go to the tensor-core kernel unless xnor_b200_set_tuning pinned the route.
	{
		const int route = tuning().gemm_route;
		const bool use_tc = sum_signs || ((route == XNOR_B200_ROUTE_AUTO) ? tc_gemm_eligible(M, n_total, K) : (route == XNOR_B200_ROUTE_TENSOR));
		if (use_tc && !(extra != nullptr && (extra->planes != nullptr || extra->masks != nullptr)))
		{
			return launch_xnor_gemm_tc(M, n_total, n_per_image, K, A, lda_words, B, ldb_words, C, ldc, mean_arr, bias, leaky,
					shortcut_in, shortcut_out, counts, stream, signs, extras ? extra : nullptr);
		}
	}

	// Short rows on a small problem: one pixel per thread, no tiling (latency, not throughput, is the issue there).
	const bool from_planes = (p.x.planes != nullptr || p.x.masks != nullptr);
	if (counts == nullptr && shortcut_out == nullptr && short_k_problem(M, n_total, p.kw, from_planes)
			&& (((uintptr_t)A | (uintptr_t)B) & 15u) == 0 && lda_words % 4 == 0 && ldb_words % 4 == 0)
	{
		switch ((K + 31) / 32)                              // K words that carry data: 1..8
		{
			case 1: return launch_smallk<1, 1>(p, stream);
			case 2: return launch_smallk<1, 2>(p, stream);
			case 3: return launch_smallk<1, 3>(p, stream);
			case 4: return launch_smallk<1, 4>(p, stream);
			case 5: return launch_smallk<2, 1>(p, stream);
			case 6: return launch_smallk<2, 2>(p, stream);
			case 7: return launch_smallk<2, 3>(p, stream);
			default: return launch_smallk<2, 4>(p, stream);
		}
	}

	if (from_planes) { return XNOR_B200_ERR_INVALID; }      // only the short-K kernel builds rows from planes

	const int os_ft = (counts == nullptr && shortcut_out == nullptr && (((uintptr_t)A | (uintptr_t)B) & 15u) == 0 && lda_words % 4 == 0 && ldb_words % 4 == 0)
			? oneshot_problem(M, n_total, p.kw, signs == nullptr && p.x.n_sinks == 0) : 0;
	if (os_ft != 0)
	{
		const int ks4 = (p.kw / 4 + OS_WARPS - 1) / OS_WARPS;      // 16-byte groups per warp
		#define XNOR_OS_CASE(N) case N: return (os_ft == 32) ? launch_oneshot<N, 32>(p, stream) : launch_oneshot<N, 16>(p, stream);
		switch (ks4)
		{
			XNOR_OS_CASE(1) XNOR_OS_CASE(2) XNOR_OS_CASE(3) XNOR_OS_CASE(4) XNOR_OS_CASE(5) XNOR_OS_CASE(6) XNOR_OS_CASE(7)
			default: return (os_ft == 32) ? launch_oneshot<8, 32>(p, stream) : launch_oneshot<8, 16>(p, stream);
		}
		#undef XNOR_OS_CASE
	}

	const int sms = sm_count();
	int best_cfg = 0, best_split = 1;
	float best = 3.0e38f;
	for (int c = 2; c < NUM_CONFIGS; ++c)
	{
		if (g_configs[c].bm > 32 && g_configs[c].bm / 2 >= M) { continue; }      // more than half the tile rows would be empty
		for (int split = 1; split <= 8; ++split)
		{
			if (split > 1 && p.kw / split < 8) { break; }                        // slices shorter than 8 words are all overhead
			const float t = estimate_cycles(g_configs[c], M, n_total, p.kw, split, sms);
			if (t < best) { best = t; best_cfg = c; best_split = split; }
		}
	}
	// xnor_b200_set_tuning may pin the tile configuration and the cluster split of the tiled kernel
	if (tuning().gemm_route == XNOR_B200_ROUTE_TILED && tuning().gemm_tile >= 1 && tuning().gemm_tile <= NUM_CONFIGS)
	{
		best_cfg = tuning().gemm_tile - 1;
		best_split = (tuning().gemm_split >= 1 && tuning().gemm_split <= 8) ? tuning().gemm_split : 1;
	}
	p.split = best_split;
	p.kw_slice = (int)round_up((size_t)(p.kw + best_split - 1) / best_split, 4);
	return g_configs[best_cfg].launch(p, stream);
}

}  // namespace xnor

using namespace xnor;

static int check_gemm_args(int M, int N, int K, const void * A, int lda, const void * B, int ldb)
{
	if (A == nullptr || B == nullptr) { return XNOR_B200_ERR_NULL; }
	if (M <= 0 || N <= 0 || K <= 0) { return XNOR_B200_ERR_INVALID; }
	if (lda < K || ldb < K || lda % 128 != 0 || ldb % 128 != 0) { return XNOR_B200_ERR_INVALID; }
	if ((((uintptr_t)A) & 15u) != 0 || (((uintptr_t)B) & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	return XNOR_B200_OK;
}

extern "C" int xnor_b200_gemm_bin_mean_transposed(int M, int N, int K,
		const uint8_t * A, int lda, const uint8_t * B, int ldb,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky_activation,
		const float * shortcut_in, float * shortcut_out, void * stream)
{
	int rc = check_gemm_args(M, N, K, A, lda, B, ldb);
	if (rc != XNOR_B200_OK) { return rc; }
	if (C == nullptr || mean_arr == nullptr) { return XNOR_B200_ERR_NULL; }
	if (ldc < N) { return XNOR_B200_ERR_INVALID; }
	if (shortcut_out != nullptr && shortcut_in == nullptr) { return XNOR_B200_ERR_NULL; }
	return launch_xnor_gemm(M, N, N, K, (const uint32_t *)A, lda / 32, (const uint32_t *)B, ldb / 32,
			C, ldc, mean_arr, bias, leaky_activation, shortcut_in, shortcut_out, nullptr, (cudaStream_t)stream);
}

extern "C" int xnor_b200_gemm_counts(int M, int N, int K, const uint8_t * A, int lda, const uint8_t * B, int ldb,
		int32_t * counts, void * stream)
{
	int rc = check_gemm_args(M, N, K, A, lda, B, ldb);
	if (rc != XNOR_B200_OK) { return rc; }
	if (counts == nullptr) { return XNOR_B200_ERR_NULL; }
	return launch_xnor_gemm(M, N, N, K, (const uint32_t *)A, lda / 32, (const uint32_t *)B, ldb / 32,
			nullptr, N, nullptr, nullptr, 0, nullptr, nullptr, counts, (cudaStream_t)stream);
}
