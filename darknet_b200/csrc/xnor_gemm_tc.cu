// XNOR GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for large layers.
//
// tcgen05.mma has no 1-bit operand kind, and the legacy mma.sync b1 path measures slower than the integer
// pipe on this GPU.  A binary dot product is nevertheless an integer GEMM: with both operands expanded to
// signed bytes holding 0 or -1,
//     D[j][i] = sum_k b_jk * a_ik = popc(B_j & A_i)            (kind::i8, s8 x s8 -> s32, exact)
//     agreeing bits = K - popc(A_i) - popc(B_j) + 2 * D[j][i]
// so the packed operands stay 1 bit per element in HBM and L2 (the same buffers the integer-pipe kernel reads)
// and are widened to bytes only inside shared memory, next to the tensor core that consumes them.
//
// Orientation: the UMMA "M" dimension (128 TMEM lanes) carries OUTPUT PIXELS, the "N" dimension (TMEM columns)
// carries FILTERS.  After tcgen05.ld each thread then owns one pixel and 32 consecutive filters per load, so
// for every filter the 32 lanes of a warp store 32 consecutive pixels: NCHW output rows are written with fully
// coalesced 128-byte stores.
//
// One CTA = 128 pixels x NF filters (NF = 128 or 256), warp-specialised:
//   warp 0            allocates TMEM; one lane issues, per 128-bit K block, 4 x tcgen05.mma.cta_group::1.kind::i8
//                     (M=128, N=NF, K=32) and a tcgen05.commit that frees the stage when the MMAs have read it;
//   warps 1..(128+NF)/32   producers: each thread owns one operand row (pixel row or filter row), keeps three
//                     K blocks of packed bits in flight from L2, expands 128 bits -> 128 bytes straight into the
//                     canonical K-major SWIZZLE_128B tile of the current stage, counts its row's set bits, and
//                     its warp arrives on the stage's "full" barrier; the same warps run the epilogue.
// Two stages per CTA and two CTAs per SM: while one CTA drains its accumulators the other keeps the tensor
// core busy.  The epilogue applies the popcount correction, mean scale, bias and leaky with the same
// two-rounding fp32 sequence as the integer-pipe kernel, so both kernels give bit-identical outputs.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in g_tc_error, all roles drop out
// of their loops, the TMEM columns are still released, and the kernel returns.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int TC_PIX = 128;                               // pixels per tile = UMMA M = TMEM lanes
constexpr int TC_STAGES = 2;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

__device__ int g_tc_error = 0;

struct TcParams
{
	const uint32_t * A;     // filters   [M][lda_words]
	const uint32_t * B;     // pixels    [n_total][ldb_words]
	int M, n_total, n_per_image, K;
	int lda_words, ldb_words;
	int kblocks;            // number of 128-bit K blocks
	float * C;
	int ldc;
	const float * mean_arr;
	const float * bias;
	int leaky;
	const float * shortcut_in;
	float * shortcut_out;
	int32_t * counts;
	uint32_t * signs;       // when set: sign bits of the output only, [img][M/32][pixel]
	int tiles_f;            // filter tiles (fastest-varying in blockIdx.x)
	GemmExtra x;            // window-major column order and direct sign sinks (all zero: none)
};

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
// another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity, volatile int * failed)
{
	const uint32_t addr = smem_u32(bar);
	for (uint32_t spin = 0; spin < TC_SPIN_LIMIT; ++spin)
	{
		uint32_t done;
		asm volatile(
			"{\n\t.reg .pred p;\n\t"
			"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
			"selp.u32 %0, 1, 0, p;\n\t}"
			: "=r"(done) : "r"(addr), "r"(parity) : "memory");
		if (done) { return true; }
		if ((spin & 1023u) == 1023u && *failed != 0) { return false; }
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

// Epilogue of a tile that only writes fp32 values (no sign words, sinks or counts): this warp's 32-filter chunks
// (share, share + shares, ...) in groups of G filters.  With a fused shortcut (SC) the loop is software-pipelined:
// the shortcut operand of group i+1 is requested before group i is computed and stored, so a thread always has
// G..2G loads in flight.  With one request per output in program order, or one batch per group and nothing in flight in
// between, the 24 warps of an SM wait a full memory latency each time and the epilogue runs at a fraction of the memory rate.
template <int G, bool SC>
__device__ __forceinline__ void epilogue_values(const TcParams & p, const int4 * s_fil, uint32_t tlane, int share, int shares,
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
			#pragma unroll
			for (int u = 0; u < G; ++u)
			{
				if (f0 + fb + u < p.M)
				{
					const int4 fi = s_fil[fb + u];                 // one broadcast 16-byte read per filter
					// 2*agree - K = (K - 2 popc(b)) - 2 popc(a) + 4 popc(a & b)
					const int dot = k_b + fi.x + 4 * (int)d[u];
					float v = __fmul_rn((float)dot, __int_as_float(fi.y));
					if (has_bias) { v = __fadd_rn(v, __int_as_float(fi.z)); }
					if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
					if (c_pix != nullptr) { c_pix[(size_t)(fb + u) * p.ldc] = v; }
					if (SC)
					{
						const float sum = __fadd_rn(sc[u], v);
						sc_out[(size_t)(fb + u) * p.ldc] = sum;
						bits |= (sum > 0.0f ? 1u : 0u) << u;
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

template <int NF>
struct TcShape
{
	static constexpr int ROWS = TC_PIX + NF;                     // operand rows per stage
	static constexpr int PRODUCER_WARPS = ROWS / 32;
	static constexpr int THREADS = 32 + ROWS;                    // warp 0 + producers
	static constexpr int PIX_TILE_BYTES = TC_PIX * 128;
	static constexpr int STAGE_BYTES = ROWS * 128;
	static constexpr int SMEM_BYTES = TC_STAGES * STAGE_BYTES + 1024;   // + slack to align the ring to 1024 bytes
};

template <int NF>
__global__ void __launch_bounds__(TcShape<NF>::THREADS, (NF == 256) ? 2 : (NF == 128) ? 3 : 4)      // co-resident CTAs: one epilogue overlaps another main loop
xnor_gemm_tc_kernel(const TcParams p)
{
	using S = TcShape<NF>;
	extern __shared__ uint8_t tc_smem_raw[];
	__shared__ uint64_t bar_full[TC_STAGES];
	__shared__ uint64_t bar_empty[TC_STAGES];
	__shared__ uint64_t bar_done;
	__shared__ uint32_t tmem_base_slot;
	__shared__ int s_pop[TC_PIX];                            // popc of every pixel row
	__shared__ int4 s_fil[NF];                               // per filter: {-2 popc(row), mean bits, bias bits, 0}
	__shared__ int s_failed_storage;
	volatile int * s_failed = &s_failed_storage;

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const uint32_t ring = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;

	const int tile_f = blockIdx.x % p.tiles_f;
	const int tile_p = blockIdx.x / p.tiles_f;
	const int f0 = tile_f * NF;
	const int n0 = tile_p * TC_PIX;

	if (tid == 0)
	{
		for (int s = 0; s < TC_STAGES; ++s)
		{
			mbar_init(&bar_full[s], S::PRODUCER_WARPS);
			mbar_init(&bar_empty[s], 1);
		}
		mbar_init(&bar_done, 1);
		s_failed_storage = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)NF) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = tmem_base_slot;

	if (warp == 0)
	{
		// ---- MMA issuer -------------------------------------------------------------------------
		if (lane == 0)
		{
			// instruction descriptor: D = s32, A = B = s8, both K-major, N = NF, M = 128
			const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NF >> 3) << 17) | ((uint32_t)(TC_PIX >> 4) << 24);
			bool ok = true;
			for (int kb = 0; kb < p.kblocks && ok; ++kb)
			{
				const int s = kb % TC_STAGES;
				ok = mbar_wait(&bar_full[s], (uint32_t)((kb / TC_STAGES) & 1), s_failed);
				if (!ok) { break; }
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t pix_addr = ring + (uint32_t)s * S::STAGE_BYTES;
				const uint32_t fil_addr = pix_addr + S::PIX_TILE_BYTES;
				#pragma unroll
				for (int k = 0; k < 4; ++k)
				{
					const uint64_t adesc = make_smem_desc(pix_addr + k * 32);
					const uint64_t bdesc = make_smem_desc(fil_addr + k * 32);
					const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
					asm volatile(
						"{\n\t.reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
						:: "r"(tmem_base), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate),
						   "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
				}
				// arrives on the stage's barrier once every MMA issued so far has finished reading shared memory
				asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
						:: "r"(smem_u32(&bar_empty[s])) : "memory");
			}
			if (ok)
			{
				asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
						:: "r"(smem_u32(&bar_done)) : "memory");
			}
		}
		__syncwarp();
	}
	else
	{
		// ---- producers ----------------------------------------------------------------------------
		const int r = tid - 32;                               // operand row of this thread within the stage
		const bool is_pix = r < TC_PIX;
		const int row_in_tile = is_pix ? r : r - TC_PIX;
		const bool row_ok = is_pix ? (n0 + row_in_tile < p.n_total) : (f0 + row_in_tile < p.M);
		const uint4 * src = reinterpret_cast<const uint4 *>(
				is_pix ? p.B + (size_t)(row_ok ? n0 + row_in_tile : 0) * p.ldb_words
				       : p.A + (size_t)(row_ok ? f0 + row_in_tile : 0) * p.lda_words);
		// byte address of this thread's row in stage 0, swizzle term folded in
		const uint32_t row_swz0 = (ring + (is_pix ? 0u : (uint32_t)S::PIX_TILE_BYTES) + (uint32_t)row_in_tile * 128u)
				^ ((uint32_t)(row_in_tile & 7) << 4);
		const uint4 zero4 = make_uint4(0, 0, 0, 0);
		uint4 w0 = (row_ok && 0 < p.kblocks) ? __ldg(src + 0) : zero4;
		uint4 w1 = (row_ok && 1 < p.kblocks) ? __ldg(src + 1) : zero4;
		uint4 w2 = (row_ok && 2 < p.kblocks) ? __ldg(src + 2) : zero4;
		int pop = 0;
		bool ok = true;
		for (int kb = 0; kb < p.kblocks; ++kb)
		{
			const int s = kb % TC_STAGES;
			const uint4 cur = w0;
			w0 = w1;
			w1 = w2;
			w2 = (row_ok && kb + 3 < p.kblocks) ? __ldg(src + kb + 3) : zero4;
			if (kb >= TC_STAGES)
			{
				// the MMAs that read this stage (issued STAGES blocks ago) must have completed
				ok = mbar_wait(&bar_empty[s], (uint32_t)((kb / TC_STAGES - 1) & 1), s_failed);
				if (!ok) { break; }
			}
			expand_row(row_swz0 + (uint32_t)s * S::STAGE_BYTES, cur);
			pop += __popc(cur.x) + __popc(cur.y) + __popc(cur.z) + __popc(cur.w);
			// generic-proxy writes -> visible to the tensor core's async proxy; then one arrival per warp
			asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
			__syncwarp();
			if (lane == 0) { mbar_arrive(&bar_full[s]); }
		}
		if (is_pix)
		{
			s_pop[row_in_tile] = pop;
		}
		else
		{
			const int f = f0 + row_in_tile;
			const float mean = (f < p.M && p.mean_arr != nullptr) ? __ldg(p.mean_arr + f) : 0.0f;
			const float bias = (f < p.M && p.bias != nullptr) ? __ldg(p.bias + f) : 0.0f;
			s_fil[row_in_tile] = make_int4(-2 * pop, __float_as_int(mean), __float_as_int(bias), 0);
		}
	}

	// ---- everyone: wait for the accumulators ----------------------------------------------------------
	mbar_wait(&bar_done, 0, s_failed);
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const bool failed = (*s_failed != 0);

	if (!failed && warp != 0)
	{
		// A warp may read TMEM lanes 32*(warp%4) .. +31.  The producer warps 1..PRODUCER_WARPS cover every lane
		// quarter PRODUCER_WARPS/4 times; warps sharing a quarter interleave over the 32-column chunks.
		const int quarter = warp & 3;
		constexpr int SHARES = S::PRODUCER_WARPS / 4;
		// 0 .. SHARES - 1; the odd producer warps of the narrow tiles (5 or 6 producer warps) have nothing left to read
		const int share = ((warp - 1) >> 2) < SHARES ? ((warp - 1) >> 2) : NF;
		const int pix_local = quarter * 32 + lane;
		const int col = n0 + pix_local;                       // global pixel (column of C)
		const bool col_ok = col < p.n_total;
		const int img = col_ok ? col / p.n_per_image : 0;
		const int pixcol = col_ok ? col - img * p.n_per_image : 0;
		const int pix = col_to_pixel(p.x, pixcol);
		const int k_b = p.K - 2 * s_pop[pix_local];
		const bool has_bias = (p.bias != nullptr);
		const size_t pix_off = ((size_t)img * p.M + f0) * p.ldc + pix;    // element (first filter of the tile, this pixel)
		float * c_pix = (p.C != nullptr) ? p.C + pix_off : nullptr;
		float * sc_out = (p.shortcut_out != nullptr) ? p.shortcut_out + pix_off : nullptr;
		const float * sc_in = (p.shortcut_in != nullptr) ? p.shortcut_in + pix_off : nullptr;
		const bool values_only = (p.signs == nullptr && p.x.n_sinks == 0 && p.counts == nullptr);
		if (values_only)
		{
			const int my_chunks = (share < NF / 32) ? (NF / 32 - share + SHARES - 1) / SHARES : 0;
			const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
			if (sc_in != nullptr)
			{
				uint32_t * sum_words = (p.x.sum_signs != nullptr)
						? p.x.sum_signs + ((size_t)img * (p.M >> 5) + (f0 >> 5)) * p.n_per_image + pix : nullptr;
				uint32_t * row_words = (p.x.sum_rows != nullptr)
						? p.x.sum_rows + ((size_t)img * p.n_per_image + pix) * p.x.sum_ldw + (f0 >> 5) : nullptr;
				epilogue_values<16, true>(p, s_fil, tlane, share, SHARES, my_chunks, f0, k_b, col_ok, c_pix, sc_in, sc_out, sum_words, p.n_per_image,
						row_words);
			}
			else { epilogue_values<32, false>(p, s_fil, tlane, share, SHARES, my_chunks, f0, k_b, col_ok, c_pix, nullptr, nullptr); }
		}
		#pragma unroll 1
		for (int chunk = values_only ? NF : share; chunk < NF / 32; chunk += SHARES)
		{
			uint32_t d[32];
			const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(chunk * 32);
			asm volatile(
				"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
				"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
				"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
				: "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
				  "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]),
				  "=r"(d[16]), "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]),
				  "=r"(d[24]), "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
				: "r"(taddr) : "memory");
			asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
			const int fbase = chunk * 32;
			if (p.signs != nullptr || p.x.n_sinks > 0)
			{
				// the 32 filters of this chunk are exactly one channel-packed word of this thread's pixel
				uint32_t word = 0;
				if (col_ok && f0 + fbase < p.M)
				{
					#pragma unroll
					for (int j = 0; j < 32; ++j)
					{
						const int4 fi = s_fil[fbase + j];
						float v = __fmul_rn((float)(k_b + fi.x + 4 * (int)d[j]), __int_as_float(fi.y));
						if (has_bias) { v = __fadd_rn(v, __int_as_float(fi.z)); }
						word |= (v > 0.0f ? 1u : 0u) << j;
					}
				}
				const int mw = (f0 + fbase) >> 5;
				const bool word_ok = col_ok && f0 + fbase < p.M;
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
						p.counts[(size_t)(f0 + fbase + j) * p.n_total + col] = (k_b + s_fil[fbase + j].x + 4 * (int)d[j] + p.K) >> 1;
					}
				}
				continue;
			}
			float * out = c_pix + (size_t)fbase * p.ldc;
			#pragma unroll
			for (int j = 0; j < 32; ++j)
			{
				if (f0 + fbase + j < p.M)
				{
					const int4 fi = s_fil[fbase + j];
					const int dot = k_b + fi.x + 4 * (int)d[j];
					float v = __fmul_rn((float)dot, __int_as_float(fi.y));
					if (has_bias) { v = __fadd_rn(v, __int_as_float(fi.z)); }
					if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
					out[(size_t)j * p.ldc] = v;
					if (sc_out != nullptr) { sc_out[(size_t)(fbase + j) * p.ldc] = __fadd_rn(__ldg(sc_in + (size_t)(fbase + j) * p.ldc), v); }
				}
			}
		}
	}
	else if (failed && tid == 0)
	{
		atomicExch(&g_tc_error, 1);
	}

	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 0)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)NF) : "memory");
	}
}

bool tc_gemm_eligible(int M, int n_total, int K)
{
	// The faster of two estimates fitted to measurements on B200 (batch 8..64 layer shapes) decides:
	//   tensor-core kernel: ~7 us of fixed cost (launch with 100+ KB of shared memory, TMEM allocation, pipeline fill,
	//                       drain) + per tile 0.6 us per 128-bit K block and 4 us of epilogue for 256-filter tiles (0.33 + 2.5,
	//                       0.25 + 2.0, 0.2 + 1.4 for 128, 64 and 32 filters), times the tiles the busiest SM gets (co-resident
	//                       CTAs share the SM's shared-memory bandwidth);
	//   integer kernel:     ~4 us + binary ops (over the K words it actually walks) at 250 T/s + 2 us per million outputs
	//                       (index arithmetic and stores of its epilogue, which dominate when K is short: 1x1 layers
	//                       over 64..256 channels at large batch run 1.3-2x faster on the tensor-core kernel).
	if (M < 16 || K < 64) { return false; }
	const int nf = (M > 128) ? 256 : (M > 64) ? 128 : (M > 32) ? 64 : 32;
	const long long tiles = (long long)((M + nf - 1) / nf) * ((n_total + TC_PIX - 1) / TC_PIX);
	const double kb = (double)((K + 127) / 128);
	const double per_tile = (nf == 256) ? 0.6 * kb + 4.0 : (nf == 128) ? 0.33 * kb + 2.5 : (nf == 64) ? 0.25 * kb + 2.0 : 0.2 * kb + 1.4;
	double load = (double)tiles / (double)sm_count();
	if (nf == 256) { load = (double)((tiles + sm_count() - 1) / sm_count()); }
	if (load < 1.0) { load = 1.0; }
	const double t_tc = 7.0 + per_tile * load;
	const double k_int = (double)(((K + 31) / 32 + 3) / 4 * 4 * 32);       // the integer kernel walks whole 16-byte groups of K words
	const double t_int = 4.0 + 2.0 * (double)M * (double)n_total * k_int / 250.0e6 + (double)M * (double)n_total / 500.0e3;
	return t_tc < t_int;
}

template <int NF>
static int launch_tc(TcParams & p, cudaStream_t stream)
{
	using S = TcShape<NF>;
	p.tiles_f = (p.M + NF - 1) / NF;
	const long long grid = (long long)p.tiles_f * ((p.n_total + TC_PIX - 1) / TC_PIX);
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	int rc = ensure_dynamic_smem((const void *)xnor_gemm_tc_kernel<NF>, S::SMEM_BYTES);
	if (rc != XNOR_B200_OK) { return rc; }
	xnor_gemm_tc_kernel<NF><<<(unsigned)grid, S::THREADS, S::SMEM_BYTES, stream>>>(p);
	return check_launch();
}

int launch_xnor_gemm_tc(int M, int n_total, int n_per_image, int K,
		const uint32_t * A, int lda_words, const uint32_t * B, int ldb_words,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky,
		const float * shortcut_in, float * shortcut_out, int32_t * counts, cudaStream_t stream, uint32_t * signs,
		const GemmExtra * extra)
{
	TcParams p;
	p.x = GemmExtra();
	if (extra != nullptr) { p.x = *extra; }
	if (p.x.out_w <= 0) { p.x.out_w = 1; }
	if (p.x.planes != nullptr || p.x.masks != nullptr) { return XNOR_B200_ERR_INVALID; }
	p.signs = signs;
	p.A = A; p.B = B;
	p.M = M; p.n_total = n_total; p.n_per_image = n_per_image; p.K = K;
	p.lda_words = lda_words; p.ldb_words = ldb_words;
	p.kblocks = (K + 127) / 128;
	p.C = C; p.ldc = ldc; p.mean_arr = mean_arr; p.bias = bias; p.leaky = leaky;
	p.shortcut_in = shortcut_in; p.shortcut_out = shortcut_out; p.counts = counts;
	if (M > 128) { return launch_tc<256>(p, stream); }
	if (M > 64) { return launch_tc<128>(p, stream); }
	return (M > 32) ? launch_tc<64>(p, stream) : launch_tc<32>(p, stream);
}

int read_tc_error(int * out, bool clear)
{
	int v = 0;
	cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
	if (e != cudaSuccess) { return cuda_fail(e); }
	if (clear && v != 0)
	{
		const int zero = 0;
		e = cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
		if (e != cudaSuccess) { return cuda_fail(e); }
	}
	*out = v;
	return XNOR_B200_OK;
}

}  // namespace xnor
