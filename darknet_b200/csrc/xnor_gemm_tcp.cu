// Persistent tcgen05 XNOR GEMM for large layers (more than 64 filters): one CTA per SM walks over 128-pixel x NF-filter
// tiles (NF = 256 or 128); the same arithmetic as the one-tile-per-CTA kernel in xnor_gemm_tc.cu (binary dot product =
// integer GEMM over bytes holding 0 / -1, kind::i8, exact int32 accumulators in TMEM), re-shaped so that the tensor pipe
// never waits for an epilogue and nobody waits for global memory:
//
//   warp  8        TMA producer: one lane brings the packed bit rows of the tile -- 128 pixel rows and NF filter rows, two
//                  128-bit K blocks (32 bytes) per row -- into a ring of raw stages with cp.async.bulk.tensor.2d (plain, no
//                  multicast; rows past the end of a matrix arrive as zeros) and mbarrier expect_tx;
//   warps 10..     expanders, one operand row per thread: raw stage -> registers -> 128 bits widened to 128 bytes straight into
//                  the K-major SWIZZLE_128B tile of the next free expanded stage, popcount of the row on the side;
//   warp  9        issuer: per K block 4 x tcgen05.mma.cta_group::1.kind::i8 (M=128, N=NF, K=32) into one of TWO accumulator
//                  buffers in TMEM, tcgen05.commit frees the expanded stage, a last commit per tile hands the buffer over;
//   warps 0..7     epilogue: tcgen05.ld of the finished buffer, popcount correction, mean scale, bias, leaky, shortcut, sign
//                  words and sinks (tc_common.cuh), while the issuer already fills the other buffer with the next tile.
//
// Every wait on an mbarrier is bounded.  When one runs out, every role leaves its loops, the producer waits (bounded) for the
// copies it still has in flight, the issuer for its MMAs, the tensor memory is released, a status word is set, and the kernel
// returns by itself.
#include "tc_common.cuh"

#include <cuda.h>       // CUtensorMap and its enums; the encoder itself is fetched through cudaGetDriverEntryPoint

#include <mutex>

namespace xnor
{

constexpr int TP_EPI_WARPS = 8;
constexpr int TP_RAW_KB = 2;                  // 128-bit K blocks per raw stage: 32 bytes per operand row
constexpr int TP_RAW_STAGES = 4;
constexpr int TP_FIRST_EXP_WARP = TP_EPI_WARPS + 2;

template <int NF>
struct TpShape
{
	static constexpr int ROWS = TC_PIX + NF;
	static constexpr int EXP_WARPS = ROWS / 32;
	static constexpr int THREADS = (TP_FIRST_EXP_WARP + EXP_WARPS) * 32;
	static constexpr int EXP_STAGES = (NF == 256) ? 3 : 4;
	// The expander warps form GROUPS groups; group g widens the K blocks number g, g + GROUPS, ... (all rows of them, several
	// rows per thread), so GROUPS K blocks are in the making at any time and a group pays the fixed cost of a hand-over
	// (waits, proxy fence, arrival) once per GROUPS K blocks.
	static constexpr int GROUPS = EXP_STAGES;
	static constexpr int WARPS_PER_GROUP = EXP_WARPS / GROUPS;
	static constexpr int GROUP_THREADS = WARPS_PER_GROUP * 32;             // ROWS == GROUPS * GROUP_THREADS
	static constexpr int EXP_STAGE_BYTES = ROWS * 128;
	static constexpr int PIX_TILE_BYTES = TC_PIX * 128;
	static constexpr int RAW_STAGE_BYTES = ROWS * 16 * TP_RAW_KB;
	static constexpr int RAW_PIX_BYTES = TC_PIX * 16 * TP_RAW_KB;
	static constexpr int SMEM_BYTES = EXP_STAGES * EXP_STAGE_BYTES + TP_RAW_STAGES * RAW_STAGE_BYTES + 1024;   // + slack to align to 1024
	static constexpr int TMEM_COLS = 2 * NF;
	static_assert(EXP_WARPS % GROUPS == 0 && ROWS == GROUPS * GROUP_THREADS, "rows must divide evenly over the groups");
};

// Wait that does not look at the CTA's failure flag (used while draining on the way out).
__device__ __forceinline__ bool mbar_wait_plain(uint64_t * bar, uint32_t parity, uint32_t limit)
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
	}
	return false;
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// One 2-D box of a row-major byte matrix -> shared memory; x = byte offset inside the rows (a multiple of 16), y = first row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap * map, int x, int y, uint64_t * bar)
{
	asm volatile(
		"cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
		:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// 16 bits -> 16 bytes, 0x00 or 0xFF each, with four byte-permutes and one shift: PRMT picks every output byte from an
// 8-byte pool by the low three bits of a selector nibble taken from the packed word itself.  Three pools answer "is bit 0 /
// bit 1 / bit 2 of the nibble set" for the same selector; bit 3 of a nibble is PRMT's sign-replication flag, harmless for
// 0x00 / 0xFF bytes, and is read through a shifted selector.  Word q of the result holds bits q, q+4, q+8, q+12 of the
// group: a permutation of K inside the 16-byte chunk that both operands share, so every dot product is unchanged.
__device__ __forceinline__ uint4 expand16p(uint32_t sel)
{
	uint4 v;
	v.x = __byte_perm(0xFF00FF00u, 0xFF00FF00u, sel);
	v.y = __byte_perm(0xFFFF0000u, 0xFFFF0000u, sel);
	v.z = __byte_perm(0x00000000u, 0xFFFFFFFFu, sel);
	v.w = __byte_perm(0xFF00FF00u, 0xFF00FF00u, sel >> 3);
	return v;
}

// One row of one K block: 128 bits -> 128 bytes at the row's place in a K-major SWIZZLE_128B tile (see expand_row).
__device__ __forceinline__ void expand_row_p(uint32_t row_swz, const uint4 w)
{
	const uint32_t words[4] = {w.x, w.y, w.z, w.w};
	#pragma unroll
	for (int c = 0; c < 8; ++c)
	{
		const uint4 v = expand16p((c & 1) ? (words[c >> 1] >> 16) : words[c >> 1]);
		asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
				:: "r"(row_swz ^ (uint32_t)(c << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
	}
}

template <int NF>
__global__ void __launch_bounds__(TpShape<NF>::THREADS, 1)
xnor_gemm_tcp_kernel(const TcParams p, const __grid_constant__ CUtensorMap map_pix, const __grid_constant__ CUtensorMap map_fil)
{
	using S = TpShape<NF>;
	extern __shared__ uint8_t tp_smem_raw[];
	__shared__ uint64_t raw_full[TP_RAW_STAGES];
	__shared__ uint64_t raw_empty[TP_RAW_STAGES];
	__shared__ uint64_t exp_full[S::EXP_STAGES];
	__shared__ uint64_t exp_empty[S::EXP_STAGES];
	__shared__ uint64_t acc_full[2];
	__shared__ uint64_t acc_empty[2];
	__shared__ uint64_t meta_full[2];
	__shared__ uint64_t comb_full[2];
	__shared__ uint64_t drain_bar;
	__shared__ uint32_t tmem_base_slot;
	__shared__ int s_part[2][S::GROUPS][S::ROWS];             // popc of every operand row over the K blocks of one group
	__shared__ int s_pop[2][TC_PIX];                          // popc of every pixel row, per accumulator buffer
	__shared__ __align__(16) int s_fil[2][3][NF];             // per filter: -2 popc(row) | mean bits | bias bits
	__shared__ int s_failed_storage;
	volatile int * s_failed = &s_failed_storage;

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const uint32_t exp_base = (smem_u32(tp_smem_raw) + 1023u) & ~1023u;
	const uint32_t raw_base = exp_base + (uint32_t)(S::EXP_STAGES * S::EXP_STAGE_BYTES);
	const uint32_t limit = p.spin_limit;
	const int chunks = (p.kblocks + TP_RAW_KB - 1) / TP_RAW_KB;

	if (tid == 0)
	{
		for (int s = 0; s < TP_RAW_STAGES; ++s)
		{
			mbar_init(&raw_full[s], 1);
			mbar_init(&raw_empty[s], TP_RAW_KB * S::WARPS_PER_GROUP);        // one arrival per K block slot and warp of its group
		}
		for (int s = 0; s < S::EXP_STAGES; ++s)
		{
			mbar_init(&exp_full[s], S::WARPS_PER_GROUP);
			mbar_init(&exp_empty[s], 1);
		}
		for (int b = 0; b < 2; ++b)
		{
			mbar_init(&acc_full[b], 1);
			mbar_init(&acc_empty[b], TP_EPI_WARPS);
			mbar_init(&meta_full[b], S::EXP_WARPS);
			mbar_init(&comb_full[b], TP_EPI_WARPS);
		}
		mbar_init(&drain_bar, 1);
		s_failed_storage = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == TP_EPI_WARPS + 1)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = tmem_base_slot;

	if (warp < TP_EPI_WARPS)
	{
		// ---- epilogue warps: two per TMEM lane quarter, interleaved over the 32-column chunks ----------------------
		const int quarter = warp & 3;
		const int share = warp >> 2;
		// this thread adds up the per-group popcounts of pixel row `tid` (tid < 128) and of one filter row
		const int my_f = (tid >= TC_PIX) ? tid - TC_PIX : tid + TC_PIX;
		int it = 0;
		for (int t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it)
		{
			const int buf = it & 1;
			const uint32_t ph = (uint32_t)((it >> 1) & 1);
			const int f0 = (t % p.tiles_f) * NF;
			const int n0 = (t / p.tiles_f) * TC_PIX;
			const bool f_ok = my_f < NF && f0 + my_f < p.M;
			const float mean = (f_ok && p.mean_arr != nullptr) ? __ldg(p.mean_arr + f0 + my_f) : 0.0f;
			const float bias = (f_ok && p.bias != nullptr) ? __ldg(p.bias + f0 + my_f) : 0.0f;
			if (!mbar_wait<64>(&meta_full[buf], ph, s_failed, limit)) { break; }
			if (tid < TC_PIX)
			{
				int sum = 0;
				#pragma unroll
				for (int g = 0; g < S::GROUPS; ++g) { sum += s_part[buf][g][tid]; }
				s_pop[buf][tid] = sum;
			}
			if (my_f < NF)
			{
				int sum = 0;
				#pragma unroll
				for (int g = 0; g < S::GROUPS; ++g) { sum += s_part[buf][g][TC_PIX + my_f]; }
				s_fil[buf][0][my_f] = -2 * sum;
				s_fil[buf][1][my_f] = __float_as_int(mean);
				s_fil[buf][2][my_f] = __float_as_int(bias);
			}
			__syncwarp();
			if (lane == 0) { mbar_arrive(&comb_full[buf]); }
			if (!mbar_wait<32>(&comb_full[buf], ph, s_failed, limit)) { break; }
			if (!mbar_wait<128>(&acc_full[buf], ph, s_failed, limit)) { break; }
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			epilogue_tile<NF>(p, s_pop[buf], FilterConsts{&s_fil[buf][0][0], NF}, tmem_base + (uint32_t)(buf * NF), quarter, lane, share, TP_EPI_WARPS / 4, f0, n0);
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
			__syncwarp();
			if (lane == 0) { mbar_arrive(&acc_empty[buf]); }
		}
	}
	else if (warp == TP_EPI_WARPS)
	{
		// ---- TMA producer -------------------------------------------------------------------------------------
		if (lane == 0)
		{
			uint32_t rc = 0;                                  // raw chunks issued so far
			bool ok = true;
			for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x)
			{
				const int f0 = (t % p.tiles_f) * NF;
				const int n0 = (t / p.tiles_f) * TC_PIX;
				for (int c = 0; c < chunks; ++c, ++rc)
				{
					const uint32_t rs = rc % TP_RAW_STAGES;
					if (rc >= TP_RAW_STAGES)
					{
						ok = mbar_wait<64>(&raw_empty[rs], (rc / TP_RAW_STAGES - 1) & 1u, s_failed, limit);
						if (!ok) { break; }
					}
					const uint32_t dst = raw_base + rs * (uint32_t)S::RAW_STAGE_BYTES;
					mbar_expect_tx(&raw_full[rs], (uint32_t)S::RAW_STAGE_BYTES);
					tma_load_2d(dst, &map_pix, c * 16 * TP_RAW_KB, n0, &raw_full[rs]);
					tma_load_2d(dst + (uint32_t)S::RAW_PIX_BYTES, &map_fil, c * 16 * TP_RAW_KB, f0, &raw_full[rs]);
				}
			}
			// no copy of this CTA may still be in flight when it exits: wait for the newest chunk of every stage
			for (uint32_t s = 0; s < (uint32_t)TP_RAW_STAGES && s < rc; ++s)
			{
				const uint32_t last = ((rc - 1 - s) / TP_RAW_STAGES) * TP_RAW_STAGES + s;       // newest chunk index congruent to s
				mbar_wait_plain(&raw_full[s], (last / TP_RAW_STAGES) & 1u, limit);
			}
		}
		__syncwarp();
	}
	else if (warp == TP_EPI_WARPS + 1)
	{
		// ---- MMA issuer -------------------------------------------------------------------------------------------
		if (lane == 0)
		{
			// instruction descriptor: D = s32, A = B = s8, both K-major, N = NF, M = 128
			const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NF >> 3) << 17) | ((uint32_t)(TC_PIX >> 4) << 24);
			uint32_t ec = 0;                                  // K blocks consumed so far
			bool ok = true;
			int it = 0;
			for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it)
			{
				const int buf = it & 1;
				if (it >= 2)
				{
					ok = mbar_wait<64>(&acc_empty[buf], (uint32_t)(((it >> 1) - 1) & 1), s_failed, limit);
					if (!ok) { break; }
				}
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t acc = tmem_base + (uint32_t)(buf * NF);
				for (int kb = 0; kb < p.kblocks; ++kb, ++ec)
				{
					const uint32_t es = ec % S::EXP_STAGES;
					ok = mbar_wait<20>(&exp_full[es], (ec / S::EXP_STAGES) & 1u, s_failed, limit);
					if (!ok) { break; }
					asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
					const uint32_t pix_addr = exp_base + es * (uint32_t)S::EXP_STAGE_BYTES;
					// 32 bytes further along K inside the 128-byte swizzle atom = +2 in the descriptor's address field
					const uint64_t adesc0 = make_smem_desc(pix_addr);
					const uint64_t bdesc0 = make_smem_desc(pix_addr + S::PIX_TILE_BYTES);
					#pragma unroll
					for (int k = 0; k < 4; ++k)
					{
						const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
						asm volatile(
							"{\n\t.reg .pred p;\n\t"
							"setp.ne.b32 p, %4, 0;\n\t"
							"tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
							:: "r"(acc), "l"(adesc0 + (uint64_t)(2 * k)), "l"(bdesc0 + (uint64_t)(2 * k)), "r"(idesc), "r"(accumulate),
							   "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
					}
					// arrives on the stage's barrier once every MMA issued so far has finished reading shared memory
					asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
							:: "r"(smem_u32(&exp_empty[es])) : "memory");
				}
				if (ok)
				{
					asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
							:: "r"(smem_u32(&acc_full[buf])) : "memory");
				}
			}
			if (!ok)
			{
				// leaving early: the MMAs already issued must have finished before the tensor memory is released
				asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
						:: "r"(smem_u32(&drain_bar)) : "memory");
				mbar_wait_plain(&drain_bar, 0, limit);
			}
		}
		__syncwarp();
	}
	else
	{
		// ---- expanders ----------------------------------------------------------------------------------------------
		constexpr int G = S::GROUPS;
		const int ew = warp - TP_FIRST_EXP_WARP;
		const int grp = ew / S::WARPS_PER_GROUP;
		const int gt = (ew - grp * S::WARPS_PER_GROUP) * 32 + lane;      // thread inside the group; its rows: gt, gt + GROUP_THREADS, ...
		const bool withhold = (p.withhold != 0 && ew == 0);
		uint32_t rc = 0, ec = 0;                              // raw chunks and K blocks passed so far (every warp counts all of them)
		bool ok = true;
		int it = 0;
		for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it)
		{
			int pop[G];
			#pragma unroll
			for (int i = 0; i < G; ++i) { pop[i] = 0; }
			for (int c = 0; c < chunks && ok; ++c, ++rc)
			{
				const uint32_t rs = rc % TP_RAW_STAGES;
				const uint32_t raw_stage = raw_base + rs * (uint32_t)S::RAW_STAGE_BYTES;
				bool have_raw = false;
				#pragma unroll
				for (int j = 0; j < TP_RAW_KB; ++j)
				{
					// slot j of the chunk holds K block c * RAW_KB + j of the tile, or nothing at the odd end of a row; its owner
					// is the group whose turn it is, and an empty slot still needs the owner's arrival on the raw stage
					const bool real = c * TP_RAW_KB + j < p.kblocks;
					if ((int)(ec % G) != grp)
					{
						if (real) { ++ec; }
						continue;
					}
					if (!have_raw)
					{
						ok = mbar_wait<32>(&raw_full[rs], (rc / TP_RAW_STAGES) & 1u, s_failed, limit);
						if (!ok) { break; }
						have_raw = true;
					}
					uint4 w[G];
					if (real)
					{
						#pragma unroll
						for (int i = 0; i < G; ++i)
						{
							asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
									: "=r"(w[i].x), "=r"(w[i].y), "=r"(w[i].z), "=r"(w[i].w)
									: "r"(raw_stage + (uint32_t)((gt + i * S::GROUP_THREADS) * 16 * TP_RAW_KB + j * 16)) : "memory");
						}
					}
					// the bits are in registers: this warp is through with the slot
					__syncwarp();
					if (lane == 0) { mbar_arrive(&raw_empty[rs]); }
					if (!real) { continue; }
					const uint32_t es = ec % S::EXP_STAGES;
					if (ec >= (uint32_t)S::EXP_STAGES)
					{
						// the MMAs that read this stage (issued EXP_STAGES blocks ago) must have completed
						ok = mbar_wait<32>(&exp_empty[es], (ec / S::EXP_STAGES - 1) & 1u, s_failed, limit);
						if (!ok) { break; }
					}
					const uint32_t stage = exp_base + es * (uint32_t)S::EXP_STAGE_BYTES;
					#pragma unroll
					for (int i = 0; i < G; ++i)
					{
						const int r = gt + i * S::GROUP_THREADS;          // pixel rows 0..127, then the filter rows
						expand_row_p((stage + (uint32_t)r * 128u) ^ ((uint32_t)(r & 7) << 4), w[i]);
						pop[i] += __popc(w[i].x) + __popc(w[i].y) + __popc(w[i].z) + __popc(w[i].w);
					}
					// generic-proxy writes -> visible to the tensor core's async proxy; then one arrival per warp
					asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
					__syncwarp();
					if (lane == 0 && !(withhold && ec == 0)) { mbar_arrive(&exp_full[es]); }
					++ec;
				}
			}
			if (!ok) { break; }
			// this group's share of every row's popcount; the buffer is free once the epilogue of two tiles ago is through
			const int buf = it & 1;
			if (it >= 2)
			{
				ok = mbar_wait<64>(&acc_empty[buf], (uint32_t)(((it >> 1) - 1) & 1), s_failed, limit);
				if (!ok) { break; }
			}
			#pragma unroll
			for (int i = 0; i < G; ++i) { s_part[buf][grp][gt + i * S::GROUP_THREADS] = pop[i]; }
			__syncwarp();
			if (lane == 0) { mbar_arrive(&meta_full[buf]); }
		}
	}

	// ---- everyone: release the tensor memory -----------------------------------------------------------------------
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (*s_failed != 0 && tid == 0) { atomicExch(p.status, 1); }
	if (warp == TP_EPI_WARPS + 1)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
	}
}

// ---- host side -----------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
		const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tensor_map_encoder()
{
	static std::once_flag once;
	static EncodeTiledFn fn = nullptr;
	std::call_once(once, []()
	{
		void * sym = nullptr;
		cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess
				&& q == cudaDriverEntryPointSuccess)
		{
			fn = (EncodeTiledFn)sym;
		}
	});
	return fn;
}

// Tensor map of a row-major bit matrix seen as bytes: `rows` rows of ld_bytes bytes, boxes of box_rows x 32 bytes.
static int make_row_map(CUtensorMap * map, const void * base, int rows, size_t ld_bytes, int box_rows)
{
	EncodeTiledFn enc = tensor_map_encoder();
	if (enc == nullptr) { return XNOR_B200_ERR_CUDA; }
	const cuuint64_t dims[2] = {(cuuint64_t)ld_bytes, (cuuint64_t)rows};
	const cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
	const cuuint32_t box[2] = {(cuuint32_t)(16 * TP_RAW_KB), (cuuint32_t)box_rows};
	const cuuint32_t elem[2] = {1, 1};
	const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem,
			CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS)
	{
		g_last_cuda_error = (int)cudaErrorInvalidValue;
		return XNOR_B200_ERR_CUDA;
	}
	return XNOR_B200_OK;
}

template <int NF>
static int launch_tcp(TcParams & p, cudaStream_t stream)
{
	using S = TpShape<NF>;
	p.tiles_f = (p.M + NF - 1) / NF;
	const long long tiles = (long long)p.tiles_f * ((p.n_total + TC_PIX - 1) / TC_PIX);
	if (tiles > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	p.tiles = (int)tiles;
	CUtensorMap map_pix, map_fil;
	int rc = make_row_map(&map_pix, p.B, p.n_total, (size_t)p.ldb_words * 4, TC_PIX);
	if (rc != XNOR_B200_OK) { return rc; }
	rc = make_row_map(&map_fil, p.A, p.M, (size_t)p.lda_words * 4, NF);
	if (rc != XNOR_B200_OK) { return rc; }
	rc = ensure_dynamic_smem((const void *)xnor_gemm_tcp_kernel<NF>, S::SMEM_BYTES);
	if (rc != XNOR_B200_OK) { return rc; }
	const int grid = (int)((tiles < (long long)sm_count()) ? tiles : (long long)sm_count());
	xnor_gemm_tcp_kernel<NF><<<grid, S::THREADS, S::SMEM_BYTES, stream>>>(p, map_pix, map_fil);
	return check_launch();
}

bool tcp_takes(int M) { return M > 64; }



int launch_xnor_gemm_tcp(TcParams & p, cudaStream_t stream)
{
	return (p.M > 128) ? launch_tcp<256>(p, stream) : launch_tcp<128>(p, stream);
}

}  // namespace xnor
