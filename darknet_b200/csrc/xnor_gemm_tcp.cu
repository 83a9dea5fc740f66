// Persistent tcgen05 XNOR GEMM for large layers (more than 64 filters): one CTA per SM walks over 128-pixel x 128-filter
// tiles; the same arithmetic as the one-tile-per-CTA kernel in xnor_gemm_tc.cu (binary dot product = integer GEMM over bytes
// holding 0 / -1, kind::i8, exact int32 accumulators in TMEM).  Measured on B200, a kernel that widens both operands into
// shared memory is bound by shared-memory bandwidth: per 128-bit K block the threads write as many bytes as the tensor core
// reads back, and the epilogue's own shared-memory reads queue up behind them.  So here only the FILTER operand goes
// through shared memory; the PIXEL operand is widened straight into tensor memory (tcgen05.st) and the MMA takes it from
// there, which halves the shared-memory traffic per multiply-accumulate:
//
//   warp 24        TMA producer: one lane brings the packed bit rows of the tile -- 128 pixel rows and 128 filter rows, four
//                  128-bit K blocks (64 bytes) per row -- into a ring of raw stages with cp.async.bulk.tensor.2d (plain, no
//                  multicast; rows past the end of a matrix arrive as zeros) and mbarrier expect_tx;
//   warps  8..15   pixel expanders, one pixel row per thread (warp w owns the TMEM lanes of quarter w % 4): 128 bits ->
//                  128 bytes in registers -> 32 columns of the operand ring in tensor memory;
//   warps 16..23   filter expanders, one filter row per thread: 128 bits -> 128 bytes straight into the K-major
//                  SWIZZLE_128B tile of the stage in shared memory.  Both kinds come in two groups that take the raw chunks
//                  in turn, and hand over the four K blocks of a chunk per round of waits, fences and arrivals: one warp
//                  alone needs about 200 cycles per row (measured), more than the tensor core needs per K block;
//   warp 25        issuer: per K block 4 x tcgen05.mma.cta_group::1.kind::i8 (M=128, N=128, K=32; A from tensor memory, B
//                  through a shared-memory descriptor) into one of TWO accumulator buffers, tcgen05.commit frees the stage,
//                  a last commit per tile hands the buffer to the epilogue;
//   warps 0..7     epilogue: tcgen05.ld of the finished buffer, popcount correction, mean scale, bias, leaky, shortcut, sign
//                  words and sinks (tc_common.cuh), while the issuer already fills the other buffer with the next tile.
//
// Tensor memory (512 columns): accumulators 2 x 128, pixel-operand ring 8 stages x 32 columns.
// Every wait on an mbarrier is bounded.  When one runs out, every role leaves its loops, the producer waits (bounded) for the
// copies it still has in flight, the issuer for its MMAs, the tensor memory is released, a status word is set, and the kernel
// returns by itself.
#include "tc_common.cuh"

#include <cuda.h>       // CUtensorMap and its enums; the encoder itself is fetched through cudaGetDriverEntryPoint

#include <mutex>

namespace xnor
{

constexpr int TP_NF = 128;                    // filters per tile
constexpr int TP_EPI_WARPS = 8;
constexpr int TP_GROUPS = 2;                  // expander groups: group g widens the raw chunks number g, g + TP_GROUPS, ...
constexpr int TP_PIX_WARP0 = 8;               // a multiple of 4: pixel warp w owns the TMEM lanes of quarter w % 4
constexpr int TP_FIL_WARP0 = TP_PIX_WARP0 + 4 * TP_GROUPS;
constexpr int TP_TMA_WARP = TP_FIL_WARP0 + 4 * TP_GROUPS;
constexpr int TP_MMA_WARP = TP_TMA_WARP + 1;
constexpr int TP_THREADS = (TP_MMA_WARP + 1) * 32;
constexpr int TP_RAW_KB = 2;                  // 128-bit K blocks per raw stage: 32 bytes per operand row
constexpr int TP_RAW_STAGES = 6;
constexpr int TP_STAGE_KB = 2;                // K blocks per operand stage: one wait and one commit of the issuer per stage (measured:
                                              // a wait per K block costs the tensor core 40 % of its time, one per two blocks 17 %)
constexpr int TP_STAGES = 4;                  // operand stages; per K block 16 KB of filter bytes in shared memory + 32 TMEM columns of pixel bytes
constexpr int TP_ROWS = TC_PIX + TP_NF;
constexpr int TP_SLOT_BYTES = TP_NF * 128;     // one K block of filter bytes
constexpr int TP_STAGE_BYTES = TP_STAGE_KB * TP_SLOT_BYTES;
constexpr int TP_RAW_STAGE_BYTES = TP_ROWS * 16 * TP_RAW_KB;
constexpr int TP_RAW_PIX_BYTES = TC_PIX * 16 * TP_RAW_KB;
constexpr int TP_SMEM_BYTES = TP_STAGES * TP_STAGE_BYTES + TP_RAW_STAGES * TP_RAW_STAGE_BYTES + 1024;   // + slack to align to 1024
constexpr int TP_TMEM_COLS = 512;
constexpr int TP_TMEM_A0 = 2 * TP_NF;         // first column of the pixel-operand ring

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

// One filter row of one K block: 128 bits -> 128 bytes at the row's place in a K-major SWIZZLE_128B tile (see expand_row).
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

// One pixel row of one K block: 128 bits -> 128 bytes -> 32 consecutive TMEM columns of this thread's lane.  Column 4c + q
// takes word q of 16-byte chunk c, i.e. byte k of the row sits in column k / 4 at byte k % 4: the same K order as the
// filter tile in shared memory.
__device__ __forceinline__ void expand_row_tmem(uint32_t taddr, const uint4 w)
{
	const uint32_t words[4] = {w.x, w.y, w.z, w.w};
	uint32_t r[32];
	#pragma unroll
	for (int c = 0; c < 8; ++c)
	{
		const uint4 v = expand16p((c & 1) ? (words[c >> 1] >> 16) : words[c >> 1]);
		r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
	}
	asm volatile(
		"tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
		"{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
		"%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
		:: "r"(taddr),
		   "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
		   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
		   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
		   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
		: "memory");
}

__global__ void __launch_bounds__(TP_THREADS, 1)
xnor_gemm_tcp_kernel(const TcParams p, const __grid_constant__ CUtensorMap map_pix, const __grid_constant__ CUtensorMap map_fil)
{
	constexpr int NF = TP_NF;
	extern __shared__ uint8_t tp_smem_raw[];
	__shared__ uint64_t raw_full[TP_RAW_STAGES];
	__shared__ uint64_t raw_empty[TP_RAW_STAGES];
	__shared__ uint64_t op_full[TP_STAGES];                   // both expanders' arrivals: the stage's pixel and filter bytes are in place
	__shared__ uint64_t op_empty[TP_STAGES];                  // tcgen05.commit: the MMAs that read the stage have completed
	__shared__ uint64_t acc_full[2];
	__shared__ uint64_t acc_empty[2];
	__shared__ uint64_t meta_full[2];
	__shared__ uint64_t comb_full[2];
	__shared__ uint64_t drain_bar;
	__shared__ uint32_t tmem_base_slot;
	__shared__ int s_part[2][TP_GROUPS][TP_ROWS];             // popc of every operand row over the K blocks one group widened
	__shared__ int s_pop[2][TC_PIX];                          // popc of every pixel row, per accumulator buffer
	__shared__ __align__(16) int s_fil[2][3][NF];             // per filter: -2 popc(row) | mean bits | bias bits
	__shared__ int s_failed_storage;
	volatile int * s_failed = &s_failed_storage;

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const uint32_t fil_base = (smem_u32(tp_smem_raw) + 1023u) & ~1023u;
	const uint32_t raw_base = fil_base + (uint32_t)(TP_STAGES * TP_STAGE_BYTES);
	const uint32_t limit = p.spin_limit;
	const int chunks = (p.kblocks + TP_RAW_KB - 1) / TP_RAW_KB;

	if (tid == 0)
	{
		for (int s = 0; s < TP_RAW_STAGES; ++s)
		{
			mbar_init(&raw_full[s], 1);
			mbar_init(&raw_empty[s], 8);                      // the four pixel and the four filter expander warps of one group
		}
		for (int s = 0; s < TP_STAGES; ++s)
		{
			mbar_init(&op_full[s], 8);
			mbar_init(&op_empty[s], 1);
		}
		for (int b = 0; b < 2; ++b)
		{
			mbar_init(&acc_full[b], 1);
			mbar_init(&acc_empty[b], TP_EPI_WARPS);
			mbar_init(&meta_full[b], 8 * TP_GROUPS);
			mbar_init(&comb_full[b], TP_EPI_WARPS);
		}
		mbar_init(&drain_bar, 1);
		s_failed_storage = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == TP_MMA_WARP)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)TP_TMEM_COLS) : "memory");
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
		int it = 0;
		for (int t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it)
		{
			const int buf = it & 1;
			const uint32_t ph = (uint32_t)((it >> 1) & 1);
			const int f0 = (t % p.tiles_f) * NF;
			const int n0 = (t / p.tiles_f) * TC_PIX;
			// thread `tid` of the 256 epilogue threads adds up the groups' popcounts of operand row `tid` (pixels, then filters)
			const bool is_fil = tid >= TC_PIX;
			const int f_row = f0 + tid - TC_PIX;
			const float mean = (is_fil && f_row < p.M && p.mean_arr != nullptr) ? __ldg(p.mean_arr + f_row) : 0.0f;
			const float bias = (is_fil && f_row < p.M && p.bias != nullptr) ? __ldg(p.bias + f_row) : 0.0f;
			if (!mbar_wait<512>(&meta_full[buf], ph, s_failed, limit)) { break; }
			int sum = 0;
			#pragma unroll
			for (int g = 0; g < TP_GROUPS; ++g) { sum += s_part[buf][g][tid]; }
			if (!is_fil) { s_pop[buf][tid] = sum; }
			else
			{
				s_fil[buf][0][tid - TC_PIX] = -2 * sum;
				s_fil[buf][1][tid - TC_PIX] = __float_as_int(mean);
				s_fil[buf][2][tid - TC_PIX] = __float_as_int(bias);
			}
			__syncwarp();
			if (lane == 0) { mbar_arrive(&comb_full[buf]); }
			if (!mbar_wait<32>(&comb_full[buf], ph, s_failed, limit)) { break; }
			if (!mbar_wait<512>(&acc_full[buf], ph, s_failed, limit)) { break; }
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			epilogue_tile<NF>(p, s_pop[buf], FilterConsts{&s_fil[buf][0][0], NF}, tmem_base + (uint32_t)(buf * NF), quarter, lane, share,
					TP_EPI_WARPS / 4, f0, n0);
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
			__syncwarp();
			if (lane == 0) { mbar_arrive(&acc_empty[buf]); }
		}
	}
	else if (warp == TP_TMA_WARP)
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
						ok = mbar_wait<256>(&raw_empty[rs], (rc / TP_RAW_STAGES - 1) & 1u, s_failed, limit);
						if (!ok) { break; }
					}
					const uint32_t dst = raw_base + rs * (uint32_t)TP_RAW_STAGE_BYTES;
					mbar_expect_tx(&raw_full[rs], (uint32_t)TP_RAW_STAGE_BYTES);
					tma_load_2d(dst, &map_pix, c * 16 * TP_RAW_KB, n0, &raw_full[rs]);
					tma_load_2d(dst + (uint32_t)TP_RAW_PIX_BYTES, &map_fil, c * 16 * TP_RAW_KB, f0, &raw_full[rs]);
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
	else if (warp == TP_MMA_WARP)
	{
		// ---- MMA issuer -------------------------------------------------------------------------------------------
		if (lane == 0)
		{
			// instruction descriptor: D = s32, A = B = s8, both K-major, N = NF, M = 128
			const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NF >> 3) << 17) | ((uint32_t)(TC_PIX >> 4) << 24);
			uint32_t sc = 0;                                  // operand stages consumed so far
			bool ok = true;
			int it = 0;
			for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it)
			{
				const int buf = it & 1;
				if (it >= 2)
				{
					ok = mbar_wait<128>(&acc_empty[buf], (uint32_t)(((it >> 1) - 1) & 1), s_failed, limit);
					if (!ok) { break; }
				}
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t acc = tmem_base + (uint32_t)(buf * NF);
				for (int kb0 = 0; kb0 < p.kblocks; kb0 += TP_STAGE_KB, ++sc)
				{
					const uint32_t es = sc % TP_STAGES;
					ok = mbar_wait<0>(&op_full[es], (sc / TP_STAGES) & 1u, s_failed, limit);
					if (!ok) { break; }
					asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
					const int nk = min(TP_STAGE_KB, p.kblocks - kb0);
					#pragma unroll
					for (int j = 0; j < TP_STAGE_KB; ++j)
					{
						if (j >= nk) { break; }
						// 32 bytes further along K = +2 in the shared-memory descriptor's address field, +8 TMEM columns
						const uint64_t bdesc0 = make_smem_desc(fil_base + (es * TP_STAGE_KB + j) * (uint32_t)TP_SLOT_BYTES);
						const uint32_t a0 = tmem_base + (uint32_t)(TP_TMEM_A0 + (int)(es * TP_STAGE_KB + j) * 32);
						#pragma unroll
						for (int k = 0; k < 4; ++k)
						{
							const uint32_t accumulate = (kb0 + j > 0 || k > 0) ? 1u : 0u;
							asm volatile(
								"{\n\t.reg .pred p;\n\t"
								"setp.ne.b32 p, %4, 0;\n\t"
								"tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
								:: "r"(acc), "r"(a0 + (uint32_t)(8 * k)), "l"(bdesc0 + (uint64_t)(2 * k)), "r"(idesc), "r"(accumulate),
								   "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
						}
					}
					// arrives on the stage's barrier once every MMA issued so far has finished reading its operands
					asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
							:: "r"(smem_u32(&op_empty[es])) : "memory");
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
	else if (warp >= TP_PIX_WARP0 && warp < TP_TMA_WARP)
	{
		// ---- expanders: pixel rows -> tensor memory (warps 8..15), filter rows -> shared memory (warps 16..23) -----------
		const bool is_pix = warp < TP_FIL_WARP0;
		const int grp = ((is_pix ? warp - TP_PIX_WARP0 : warp - TP_FIL_WARP0) >> 2);
		const int row = (warp & 3) * 32 + lane;               // row of the tile this thread owns
		const uint32_t raw_row = raw_base + (uint32_t)((is_pix ? row : TC_PIX + row) * 16 * TP_RAW_KB);
		const uint32_t fil_row_swz0 = (fil_base + (uint32_t)row * 128u) ^ ((uint32_t)(row & 7) << 4);     // stage 0, swizzle folded in
		const uint32_t pix_tmem0 = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)TP_TMEM_A0;   // this warp's lanes, stage 0
		const bool withhold = (p.withhold != 0 && warp == TP_PIX_WARP0);
		uint32_t rc = 0, sc = 0;                              // raw chunks and operand stages passed so far (every warp counts all of them)
		bool ok = true;
		int it = 0;
		for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it)
		{
			int pop = 0;
			for (int c = 0; c < chunks && ok; ++c, ++rc)
			{
				const int nkb = min(TP_RAW_KB, p.kblocks - c * TP_RAW_KB);      // K blocks in this chunk (fewer at the end of a row)
				const uint32_t nst = (uint32_t)(nkb + TP_STAGE_KB - 1) / TP_STAGE_KB;       // operand stages it fills
				if ((int)(rc % TP_GROUPS) != grp)
				{
					sc += nst;                                                   // the other group's chunk
					continue;
				}
				const uint32_t rs = rc % TP_RAW_STAGES;
				ok = mbar_wait<128>(&raw_full[rs], (rc / TP_RAW_STAGES) & 1u, s_failed, limit);
				if (!ok) { break; }
				uint4 w[TP_RAW_KB];
				#pragma unroll
				for (int j = 0; j < TP_RAW_KB; ++j)
				{
					asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
							: "=r"(w[j].x), "=r"(w[j].y), "=r"(w[j].z), "=r"(w[j].w)
							: "r"(raw_row + rs * (uint32_t)TP_RAW_STAGE_BYTES + (uint32_t)(j * 16)) : "memory");
				}
				// the bits are in registers: the raw stage can take the next copy
				__syncwarp();
				if (lane == 0) { mbar_arrive(&raw_empty[rs]); }
				// wait for the stages of this chunk's K blocks, widen them all, then one round of fences and arrivals
				#pragma unroll
				for (int js = 0; js < TP_RAW_KB / TP_STAGE_KB; ++js)
				{
					if (js < (int)nst && sc + js >= (uint32_t)TP_STAGES)
					{
						// the MMAs that read this stage (issued TP_STAGES stages ago) must have completed
						ok = ok && mbar_wait<128>(&op_empty[(sc + js) % TP_STAGES], ((sc + js) / TP_STAGES - 1) & 1u, s_failed, limit);
					}
				}
				if (!ok) { break; }
				// K block j of the chunk goes to slot j % STAGE_KB of stage sc + j / STAGE_KB
				if (is_pix)
				{
					asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
					#pragma unroll
					for (int j = 0; j < TP_RAW_KB; ++j)
					{
						if (j < nkb) { expand_row_tmem(pix_tmem0 + (((sc + j / TP_STAGE_KB) % TP_STAGES) * TP_STAGE_KB + j % TP_STAGE_KB) * 32u, w[j]); }
					}
					asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
					asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
				}
				else
				{
					#pragma unroll
					for (int j = 0; j < TP_RAW_KB; ++j)
					{
						if (j < nkb)
						{
							expand_row_p(fil_row_swz0 + (((sc + j / TP_STAGE_KB) % TP_STAGES) * TP_STAGE_KB + j % TP_STAGE_KB) * (uint32_t)TP_SLOT_BYTES, w[j]);
						}
					}
					// generic-proxy writes -> visible to the tensor core's async proxy
					asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
				}
				#pragma unroll
				for (int j = 0; j < TP_RAW_KB; ++j)
				{
					if (j < nkb) { pop += __popc(w[j].x) + __popc(w[j].y) + __popc(w[j].z) + __popc(w[j].w); }
				}
				__syncwarp();
				if (lane == 0)
				{
					#pragma unroll
					for (int js = 0; js < TP_RAW_KB / TP_STAGE_KB; ++js)
					{
						if (js < (int)nst && !(withhold && sc + js == 0)) { mbar_arrive(&op_full[(sc + js) % TP_STAGES]); }
					}
				}
				sc += nst;
			}
			if (!ok) { break; }
			// this group's share of the row's popcount; the buffer is free once the epilogue of two tiles ago is through
			const int buf = it & 1;
			if (it >= 2)
			{
				ok = mbar_wait<512>(&acc_empty[buf], (uint32_t)(((it >> 1) - 1) & 1), s_failed, limit);
				if (!ok) { break; }
			}
			s_part[buf][grp][is_pix ? row : TC_PIX + row] = pop;
			__syncwarp();
			if (lane == 0) { mbar_arrive(&meta_full[buf]); }
		}
	}

	// ---- everyone: release the tensor memory -----------------------------------------------------------------------
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (*s_failed != 0 && tid == 0) { atomicExch(p.status, 1); }
	if (warp == TP_MMA_WARP)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TP_TMEM_COLS) : "memory");
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

static int launch_tcp(TcParams & p, cudaStream_t stream)
{
	p.tiles_f = (p.M + TP_NF - 1) / TP_NF;
	const long long tiles = (long long)p.tiles_f * ((p.n_total + TC_PIX - 1) / TC_PIX);
	if (tiles > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	p.tiles = (int)tiles;
	CUtensorMap map_pix, map_fil;
	int rc = make_row_map(&map_pix, p.B, p.n_total, (size_t)p.ldb_words * 4, TC_PIX);
	if (rc != XNOR_B200_OK) { return rc; }
	rc = make_row_map(&map_fil, p.A, p.M, (size_t)p.lda_words * 4, TP_NF);
	if (rc != XNOR_B200_OK) { return rc; }
	rc = ensure_dynamic_smem((const void *)xnor_gemm_tcp_kernel, TP_SMEM_BYTES);
	if (rc != XNOR_B200_OK) { return rc; }
	const int grid = (int)((tiles < (long long)sm_count()) ? tiles : (long long)sm_count());
	xnor_gemm_tcp_kernel<<<grid, TP_THREADS, TP_SMEM_BYTES, stream>>>(p, map_pix, map_fil);
	return check_launch();
}

// Where the persistent kernel is the library's own choice: long rows over many filters with the plain fp32 epilogue
// (measured on B200 against the one-tile-per-CTA kernel: M=1024 N=43264 K=9216 471 vs 496 us, M=512 K=2304 level; with a
// fused shortcut or short rows the other kernel's 24 epilogue warps per SM win, e.g. 137 vs 209 us for M=256 N=100352
// K=1152 with shortcut).

int launch_xnor_gemm_tcp(TcParams & p, cudaStream_t stream)
{
	return launch_tcp(p, stream);
}

}  // namespace xnor
