// Device helpers shared by the two tcgen05 (tensor-core) XNOR GEMM kernels: bounded mbarrier waits, the bit -> byte
// expansion into the K-major SWIZZLE_128B operand layout, shared-memory and instruction descriptors, TMEM loads and the
// epilogues (popcount correction, mean scale, bias, leaky, fused shortcut, sign words and sign sinks).
#pragma once

#include "xnor_common.cuh"

namespace xnor
{

constexpr int TC_PIX = 128;                               // pixels per tile = UMMA M = TMEM lanes
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;              // default number of polls after which a barrier wait gives up

struct TcParams
{
	const uint32_t * A;     // filters   [M][lda_words]
	const uint32_t * B;     // pixels    [n_total][ldb_words]
	int M, n_total, n_per_image, K;
	int lda_words, ldb_words;
	int kblocks;            // number of K blocks (128 bits for the kind::i8 kernel, 256 bits for the kind::mxf4 kernel)
	int pad_bits;           // kind::mxf4 kernel: zero bits behind K that the K blocks cover (each counts as one agreeing position)
	float * C;
	int ldc;
	const float * mean_arr;
	const float * bias;
	int leaky;
	const float * shortcut_in;
	float * shortcut_out;
	int32_t * counts;
	uint32_t * signs;       // when set: sign bits of the output only, [img][M/32][pixel]
	int tiles_f;            // filter tiles (fastest-varying in the tile index)
	int tiles;              // persistent kernel: filter tiles x pixel tiles
	int * status;           // device word set to 1 when a bounded wait ran out
	uint32_t spin_limit;    // polls per barrier wait
	int tiles_per_image;    // persistent kernel with the staged epilogue: 128-pixel tiles per image (0: tiles over the whole batch)
	int bulk_out;           // persistent kernel: fp32 results leave through shared memory and bulk copies (1: the output, 2: the shortcut sum)
	int withhold;           // test aid: one producer arrival of the first K block is withheld (the issuer's wait then runs out)
	GemmExtra x;            // window-major column order and direct sign sinks (all zero: none)
};

// The status word of the current device (resolved once per device), the poll limit and the test switches for a launch.
int tc_fill_launch_fields(TcParams & p);

// The persistent kernel (xnor_gemm_tcp.cu).
int launch_xnor_gemm_tcp(TcParams & p, cudaStream_t stream);
// How the persistent kernel would send this call's fp32 results out through shared memory and tensor stores: 0 = not at all,
// 1 = the layer's output, 2 = the sum with a shortcut operand.
int tcp_stages_output(const TcParams & p);

// read-once data (the shortcut operand): streaming load, evicted first
__device__ __forceinline__ float ld_stream(const float * p) { return __ldcs(p); }

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t * bar)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

// Bounded wait for the phase with the given parity.  Gives up (returns false) when the limit runs out or when
// another thread of the CTA has already given up.  SLEEP_NS > 0: the warp sleeps that long between polls, so that a role
// that waits for a whole tile does not take issue slots from the warps that do the work.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity, volatile int * failed, uint32_t limit)
{
	const uint32_t addr = smem_u32(bar);
	for (uint32_t spin = 0; spin < limit; ++spin)
	{
		uint32_t done;
		asm volatile(
			"{\n\t.reg .pred p;\n\t"
			"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
			"selp.u32 %0, 1, 0, p;\n\t}"
			: "=r"(done) : "r"(addr), "r"(parity) : "memory");
		if (done) { return true; }
		if (SLEEP_NS > 0) { __nanosleep(SLEEP_NS); }
		if ((spin & 255u) == 255u && *failed != 0) { return false; }
	}
	*failed = 1;
	return false;
}

// 16 bits -> 16 bytes, each 0x00 (bit clear) or 0xFF (bit set), with one byte-permute per 4 bytes: PRMT picks
// every output byte from an 8-byte pool by a 4-bit selector taken from the packed word itself.  The pool
// alternates 0x00, 0xFF, so only the selector's lowest bit matters, and since 0x00 / 0xFF are their own sign
// replication the selector's mode bit does not matter either: no masking is needed.  Word q of the result holds
// bits q, q+4, q+8, q+12 of the group -- a permutation of K inside the 16-byte chunk that is applied identically to
// both operands and therefore leaves every dot product unchanged.  As signed bytes the values are 0 and -1, and
// (-1)*(-1) = +1, so the s8 x s8 -> s32 MMA still accumulates popc(a & b).
__device__ __forceinline__ uint4 expand16(uint32_t bits)
{
	constexpr uint32_t POOL = 0xFF00FF00u;
	uint4 v;
	v.x = __byte_perm(POOL, POOL, bits);
	v.y = __byte_perm(POOL, POOL, bits >> 1);
	v.z = __byte_perm(POOL, POOL, bits >> 2);
	v.w = __byte_perm(POOL, POOL, bits >> 3);
	return v;
}

// One row of one K block: 128 bits -> 128 bytes of a K-major tile with the 128-byte swizzle: 16-byte chunk c of
// row r lives at chunk position c ^ (r % 8) (tile base 1024-byte aligned, rows 128 bytes apart).  row_swz is
// the row's byte address with (r % 8) << 4 already XOR-ed in, so each chunk address is one XOR with a constant.
__device__ __forceinline__ void expand_row(uint32_t row_swz, const uint4 w)
{
	const uint32_t words[4] = {w.x, w.y, w.z, w.w};
	#pragma unroll
	for (int c = 0; c < 8; ++c)
	{
		const uint4 v = expand16(words[c >> 1] >> ((c & 1) * 16));
		asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
				:: "r"(row_swz ^ (uint32_t)(c << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
	}
}

// kind::mxf4 operands: 32 bits -> 32 four-bit floats (e2m1) in 16 bytes, +1.0 (0x2) where the bit is set, -1.0 (0xA) where it is
// clear: the nibble is 0xA with its sign bit cleared by the data bit.  Word q of the result takes bits q, q+4, ..., q+28 (bit
// q + 4 e lands in nibble e) -- again a permutation of K inside the chunk that both operands share.  One shift and one
// three-input logic operation per word.
__device__ __forceinline__ uint4 expand_fp4(uint32_t bits)
{
	constexpr uint32_t SIGN = 0x88888888u, MINUS_ONE = 0xAAAAAAAAu;
	uint4 v;
	v.x = ((bits << 3) & SIGN) ^ MINUS_ONE;
	v.y = ((bits << 2) & SIGN) ^ MINUS_ONE;
	v.z = ((bits << 1) & SIGN) ^ MINUS_ONE;
	v.w = (bits & SIGN) ^ MINUS_ONE;
	return v;
}

// One row of one 256-bit K block -> 128 bytes of a K-major SWIZZLE_128B tile (same placement rule as expand_row).
__device__ __forceinline__ void expand_row_fp4(uint32_t row_swz, const uint4 lo, const uint4 hi)
{
	const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
	#pragma unroll
	for (int c = 0; c < 8; ++c)
	{
		const uint4 v = expand_fp4(words[c]);
		asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
				:: "r"(row_swz ^ (uint32_t)(c << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
	}
}

// Shared-memory matrix descriptor: K-major, SWIZZLE_128B, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr)
{
	uint64_t d = 0;
	d |= (uint64_t)((addr >> 4) & 0x3FFFu);          // start address, 16-byte units
	d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major): 1
	d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
	d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
	d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
	return d;
}

// TMEM -> registers, G consecutive columns of this warp's 32 lanes
template <int G>
__device__ __forceinline__ void tmem_load(uint32_t taddr, uint32_t (&d)[G])
{
	static_assert(G == 16 || G == 32, "16 or 32 columns");
	if constexpr (G == 16)
	{
		asm volatile(
			"tcgen05.ld.sync.aligned.32x32b.x16.b32 "
			"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
			: "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
			  "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
			: "r"(taddr) : "memory");
	}
	else
	{
		asm volatile(
			"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
			"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
			"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
			: "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
			  "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]),
			  "=r"(d[16]), "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]),
			  "=r"(d[24]), "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
			: "r"(taddr) : "memory");
	}
}

// 2 * agreeing - K of one output, as a float, from its raw accumulator.
//   ACCF == false (kind::i8, operands 0 / -1, s32 accumulator d = popc(a & b)):  (K - 2 popc(b)) - 2 popc(a) + 4 d = k_b + fx + 4 d
//   ACCF == true  (kind::mxf4, operands +1 / -1 over the zero-padded rows, f32 accumulator): every position the K blocks cover
//                 behind K is a zero bit in both rows, i.e. (-1)(-1) = +1, so the value is d - pad; exact, |d| <= 2^24.
template <bool ACCF>
__device__ __forceinline__ float acc_count(uint32_t d, int k_b, int fx, float pad)
{
	if (ACCF) { return __fsub_rn(__uint_as_float(d), pad); }
	return (float)(k_b + fx + 4 * (int)d);
}

// Per-filter constants of a tile in shared memory, one array per constant so that eight consecutive filters are two 16-byte
// reads each: x = -2 popc(filter row), mean and bias as float bits.  `base` is 16-byte aligned, the arrays `nf` ints apart.
struct FilterConsts
{
	const int * base;
	int nf;
	__device__ __forceinline__ int x(int f) const { return base[f]; }
	__device__ __forceinline__ int mean(int f) const { return base[nf + f]; }
	__device__ __forceinline__ int bias(int f) const { return base[2 * nf + f]; }
	// N consecutive filters from f on (f and N multiples of 4)
	template <int N>
	__device__ __forceinline__ void load(int f, int (&fx)[N], int (&fm)[N], int (&fb)[N]) const
	{
		#pragma unroll
		for (int h = 0; h < N / 4; ++h)
		{
			const int4 a = *reinterpret_cast<const int4 *>(base + f + 4 * h);
			const int4 m = *reinterpret_cast<const int4 *>(base + nf + f + 4 * h);
			const int4 b = *reinterpret_cast<const int4 *>(base + 2 * nf + f + 4 * h);
			fx[4 * h] = a.x; fx[4 * h + 1] = a.y; fx[4 * h + 2] = a.z; fx[4 * h + 3] = a.w;
			fm[4 * h] = m.x; fm[4 * h + 1] = m.y; fm[4 * h + 2] = m.z; fm[4 * h + 3] = m.w;
			fb[4 * h] = b.x; fb[4 * h + 1] = b.y; fb[4 * h + 2] = b.z; fb[4 * h + 3] = b.w;
		}
	}
};

// Epilogue of a tile that only writes fp32 values (no sign words, sinks or counts): this warp's 32-filter chunks
// (share, share + shares, ...) in groups of G filters.  With a fused shortcut (SC) the loop is software-pipelined:
// the shortcut operand of group i+1 is requested before group i is computed and stored, so a thread always has
// G..2G loads in flight.  With one request per output in program order, or one batch per group and nothing in flight in
// between, the 24 warps of an SM wait a full memory latency each time and the epilogue runs at a fraction of the memory rate.
template <int G, bool SC, bool ACCF>
__device__ __forceinline__ void epilogue_values(const TcParams & p, const FilterConsts s_fil, uint32_t tlane, int share, int shares,
		int my_chunks, int f0, int k_b, bool col_ok, float * c_pix, const float * sc_in, float * sc_out,
		uint32_t * sum_words = nullptr, int sum_stride = 0, uint32_t * row_words = nullptr)
{
	// row_words: this pixel's row in the packed operand of the 1x1 layer that reads the sum, at the tile's first 32-filter block
	// sum_words (SC only, G == 16): word of this pixel for the tile's first 32 filters in the sign tensor of the sum, sum_stride
	// words between consecutive 32-filter blocks; the two groups of a block give the low and the high half of its word
	uint32_t word = 0;
	constexpr int PER = 32 / G;
	const int groups = my_chunks * PER;
	auto group_base = [&](int i) { return (share + (i / PER) * shares) * 32 + (i % PER) * G; };
	const bool has_bias = (p.bias != nullptr);
	float sc[SC ? G : 1];
	if (SC)
	{
		#pragma unroll
		for (int u = 0; u < G; ++u) { sc[u] = 0.0f; }
		if (groups > 0 && col_ok)
		{
			const int fb = group_base(0);
			#pragma unroll
			for (int u = 0; u < G; ++u) { if (f0 + fb + u < p.M) { sc[u] = ld_stream(sc_in + (size_t)(fb + u) * p.ldc); } }
		}
	}
	#pragma unroll 1
	for (int i = 0; i < groups; ++i)
	{
		const int fb = group_base(i);
		uint32_t d[G];
		tmem_load<G>(tlane + (uint32_t)fb, d);
		float scn[SC ? G : 1];
		if (SC)
		{
			#pragma unroll
			for (int u = 0; u < G; ++u) { scn[u] = 0.0f; }
			if (i + 1 < groups && col_ok)
			{
				const int fbn = group_base(i + 1);
				#pragma unroll
				for (int u = 0; u < G; ++u) { if (f0 + fbn + u < p.M) { scn[u] = ld_stream(sc_in + (size_t)(fbn + u) * p.ldc); } }
			}
		}
		asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
		if (col_ok)
		{
			uint32_t bits = 0;
			// NB filters at a time (eight; four beside a fused shortcut, whose operands in flight need the registers): their
			// constants are read from shared memory first, then the values are formed, then stored.  A shared-memory read behind a store through a generic pointer cannot be moved ahead of it by
			// the compiler, so one read per output in program order leaves the few epilogue warps waiting on every one.
			constexpr int NB = SC ? 4 : 8;
			const bool all_in = (f0 + fb + G <= p.M);
			const float pad = (float)p.pad_bits;
			const float slope = p.leaky ? 0.1f : 1.0f;             // leaky(v) = max(v, 0.1 v), linear(v) = max(v, v): same bits as the select
			#pragma unroll
			for (int u0 = 0; u0 < G; u0 += NB)
			{
				int fx[NB], fm[NB], fb_[NB];
				s_fil.load<NB>(fb + u0, fx, fm, fb_);                               // broadcast 16-byte reads
				float v[NB];
				#pragma unroll
				for (int j = 0; j < NB; ++j)
				{
					v[j] = __fmul_rn(acc_count<ACCF>(d[u0 + j], k_b, fx[j], pad), __int_as_float(fm[j]));
					if (has_bias) { v[j] = __fadd_rn(v[j], __int_as_float(fb_[j])); }
					v[j] = fmaxf(v[j], __fmul_rn(v[j], slope));
				}
				#pragma unroll
				for (int j = 0; j < NB; ++j)
				{
					const int u = u0 + j;
					if (all_in || f0 + fb + u < p.M)
					{
						if (c_pix != nullptr) { c_pix[(size_t)(fb + u) * p.ldc] = v[j]; }
						if (SC)
						{
							const float sum = __fadd_rn(sc[u], v[j]);
							sc_out[(size_t)(fb + u) * p.ldc] = sum;
							bits |= (sum > 0.0f ? 1u : 0u) << u;
						}
					}
				}
			}
			if (SC && G == 16 && (sum_words != nullptr || row_words != nullptr))
			{
				if ((fb & 16) == 0) { word = bits; }
				else
				{
					word |= bits << 16;
					if (f0 + fb < p.M)
					{
						if (sum_words != nullptr) { sum_words[(size_t)(fb >> 5) * sum_stride] = word; }
						if (row_words != nullptr) { row_words[fb >> 5] = word; }
					}
				}
			}
		}
		if (SC)
		{
			#pragma unroll
			for (int u = 0; u < G; ++u) { sc[u] = scn[u]; }
		}
	}
}

// One channel-packed word of sign bits (32 filters from 32 * mw on, of this thread's pixel): into the layer's sign words and
// into the operands of the consumers behind its sinks.  Every lane of the warp calls it (a pooled sink combines the four lanes
// of a 2x2 window with shuffles); word_ok = this lane's pixel and filter group exist.
__device__ __forceinline__ void emit_sign_word(const TcParams & p, uint32_t word, bool word_ok, int img, int pixcol, int pix, int col, int mw)
{
	if (p.signs != nullptr && word_ok) { p.signs[((size_t)img * (p.M >> 5) + mw) * p.n_per_image + pix] = word; }
	#pragma unroll
	for (int si = 0; si < 2; ++si)
	{
		if (si >= p.x.n_sinks) { break; }
		const SinkParams & sk = p.x.sinks[si];
		if (sk.pool != 0)
		{
			// window-major columns: lanes 4w .. 4w+3 hold one 2x2 window and share the taps of its pooled word
			uint32_t w = word;
			w |= __shfl_xor_sync(0xffffffffu, w, 1);
			w |= __shfl_xor_sync(0xffffffffu, w, 2);
			if (!word_ok) { continue; }
			const int q = pixcol >> 2;
			const int wy = q / p.x.win_w;
			const int wx = q - wy * p.x.win_w;
			for (int tap = col & 3; tap < sk.taps; tap += 4) { sink_store_tap(sk, img, wy, wx, mw, tap, w); }
		}
		else if (word_ok)
		{
			const int oy = pix / p.x.out_w;
			const int ox = pix - oy * p.x.out_w;
			const int copies = (sk.up == 2) ? 4 : 1;
			for (int t = 0; t < copies * sk.taps; ++t)
			{
				const int cp = t / sk.taps;
				const int tap = t - cp * sk.taps;
				sink_store_tap(sk, img, (sk.up == 2) ? 2 * oy + (cp >> 1) : oy, (sk.up == 2) ? 2 * ox + (cp & 1) : ox, mw, tap, word);
			}
		}
	}
}

// Epilogue of one 128-pixel x NF-filter tile for one warp.  A warp may read the TMEM lanes 32*(warp % 4) .. +31 (`quarter`);
// the `shares` warps that sit on the same quarter interleave over the tile's 32-column chunks (share, share + shares, ...).
// tmem_acc = TMEM address of the accumulator's first column at lane 0; s_pop[pixel of the tile] = popc of its row;
// s_fil = the per-filter constants of the tile (FilterConsts).
template <int NF, bool ACCF = false>
__device__ __forceinline__ void epilogue_tile(const TcParams & p, const int * s_pop, const FilterConsts s_fil, uint32_t tmem_acc,
		int quarter, int lane, int share, int shares, int f0, int n0)
{
	const int pix_local = quarter * 32 + lane;
	const int col = n0 + pix_local;                       // global pixel (column of C)
	const bool col_ok = col < p.n_total;
	const int img = col_ok ? col / p.n_per_image : 0;
	const int pixcol = col_ok ? col - img * p.n_per_image : 0;
	const int pix = col_to_pixel(p.x, pixcol);
	const int k_b = ACCF ? 0 : p.K - 2 * s_pop[pix_local];
	const float pad = (float)p.pad_bits;
	const bool has_bias = (p.bias != nullptr);
	const size_t pix_off = ((size_t)img * p.M + f0) * p.ldc + pix;    // element (first filter of the tile, this pixel)
	float * c_pix = (p.C != nullptr) ? p.C + pix_off : nullptr;
	float * sc_out = (p.shortcut_out != nullptr) ? p.shortcut_out + pix_off : nullptr;
	const float * sc_in = (p.shortcut_in != nullptr) ? p.shortcut_in + pix_off : nullptr;
	const bool values_only = (p.signs == nullptr && p.x.n_sinks == 0 && p.counts == nullptr);
	const uint32_t tlane = tmem_acc + ((uint32_t)(quarter * 32) << 16);
	if (values_only)
	{
		const int my_chunks = (share < NF / 32) ? (NF / 32 - share + shares - 1) / shares : 0;
		if (sc_in != nullptr)
		{
			uint32_t * sum_words = (p.x.sum_signs != nullptr)
					? p.x.sum_signs + ((size_t)img * (p.M >> 5) + (f0 >> 5)) * p.n_per_image + pix : nullptr;
			uint32_t * row_words = (p.x.sum_rows != nullptr)
					? p.x.sum_rows + ((size_t)img * p.n_per_image + pix) * p.x.sum_ldw + (f0 >> 5) : nullptr;
			epilogue_values<16, true, ACCF>(p, s_fil, tlane, share, shares, my_chunks, f0, k_b, col_ok, c_pix, sc_in, sc_out, sum_words, p.n_per_image,
					row_words);
		}
		else { epilogue_values<32, false, ACCF>(p, s_fil, tlane, share, shares, my_chunks, f0, k_b, col_ok, c_pix, nullptr, nullptr); }
		return;
	}
	#pragma unroll 1
	for (int chunk = share; chunk < NF / 32; chunk += shares)
	{
		uint32_t d[32];
		tmem_load<32>(tlane + (uint32_t)(chunk * 32), d);
		asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
		const int fbase = chunk * 32;
		if (p.signs != nullptr || p.x.n_sinks > 0)
		{
			// the 32 filters of this chunk are exactly one channel-packed word of this thread's pixel
			uint32_t word = 0;
			if (col_ok && f0 + fbase < p.M)
			{
				#pragma unroll
				for (int j0 = 0; j0 < 32; j0 += 8)
				{
					int fx[8], fm[8], fb_[8];
					s_fil.load<8>(fbase + j0, fx, fm, fb_);
					#pragma unroll
					for (int j = 0; j < 8; ++j)
					{
						float v = __fmul_rn(acc_count<ACCF>(d[j0 + j], k_b, fx[j], pad), __int_as_float(fm[j]));
						if (has_bias) { v = __fadd_rn(v, __int_as_float(fb_[j])); }
						word |= (v > 0.0f ? 1u : 0u) << (j0 + j);
					}
				}
			}
			emit_sign_word(p, word, col_ok && f0 + fbase < p.M, img, pixcol, pix, col, (f0 + fbase) >> 5);
			if (p.C == nullptr) { continue; }
		}
		if (!col_ok) { continue; }
		if (p.counts != nullptr)
		{
			#pragma unroll
			for (int j = 0; j < 32; ++j)
			{
				if (f0 + fbase + j < p.M)
				{
					// agreeing bits among the first K
					p.counts[(size_t)(f0 + fbase + j) * p.n_total + col] = (__float2int_rn(acc_count<ACCF>(d[j], k_b, s_fil.x(fbase + j), pad)) + p.K) >> 1;
				}
			}
			continue;
		}
		float * out = c_pix + (size_t)fbase * p.ldc;
		const float slope = p.leaky ? 0.1f : 1.0f;
		#pragma unroll
		for (int j0 = 0; j0 < 32; j0 += 8)
		{
			int fx[8], fm[8], fb_[8];
			s_fil.load<8>(fbase + j0, fx, fm, fb_);
			float v[8];
			#pragma unroll
			for (int j = 0; j < 8; ++j)
			{
				v[j] = __fmul_rn(acc_count<ACCF>(d[j0 + j], k_b, fx[j], pad), __int_as_float(fm[j]));
				if (has_bias) { v[j] = __fadd_rn(v[j], __int_as_float(fb_[j])); }
				v[j] = fmaxf(v[j], __fmul_rn(v[j], slope));
			}
			#pragma unroll
			for (int j = 0; j < 8; ++j)
			{
				if (f0 + fbase + j0 + j < p.M)
				{
					out[(size_t)(j0 + j) * p.ldc] = v[j];
					if (sc_out != nullptr) { sc_out[(size_t)(fbase + j0 + j) * p.ldc] = __fadd_rn(__ldg(sc_in + (size_t)(fbase + j0 + j) * p.ldc), v[j]); }
				}
			}
		}
	}
}

}  // namespace xnor
