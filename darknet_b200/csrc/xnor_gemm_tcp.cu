// Persistent tcgen05 XNOR GEMM: one CTA per SM walks over 128-pixel x 128-filter tiles; the same arithmetic as the
// one-tile-per-CTA kernel in xnor_gemm_tc.cu (bits widened to e2m1 +1.0 / -1.0, tcgen05.mma kind::mxf4 with both scale factors
// at 2^0, exact fp32 accumulators in TMEM), with the roles separated so that none of them waits for another more than once per
// stage and the epilogue of a tile runs under the main loop of the next:
//
//   warp 24        TMA producer: one lane brings the packed bit rows of the tile -- 128 pixel rows and 128 filter rows, one
//                  256-bit K block (32 bytes) per row and raw stage -- into a ring of raw stages with cp.async.bulk.tensor.2d
//                  (one plain copy per CTA; rows and columns past the end of a matrix arrive as zeros) and mbarrier expect_tx;
//   warps  8..15   pixel expanders, warps 16..23 filter expanders, one operand row per thread: 256 bits -> 256 four-bit
//                  values = one 128-byte row of the stage's K-major SWIZZLE_128B tile in shared memory.  Both kinds come in
//                  two groups that take the raw chunks in turn;
//   warp 25        issuer: per stage 4 x tcgen05.mma.cta_group::1.kind::mxf4.block_scale (M=128, N=128, K=64, both operands
//                  through shared-memory descriptors) into one of TWO accumulator buffers, tcgen05.commit frees the stage,
//                  a last commit per tile hands the buffer to the epilogue;
//   warps 0..7     epilogue: tcgen05.ld of the finished buffer, mean scale, bias, leaky, then either the shared epilogue of
//                  tc_common.cuh (sign words, sinks, counts, output + shortcut) or, for fp32 rows only, the staged one: values
//                  (or their sum with the shortcut operand found there) go to a [filter][pixel] staging buffer in two halves;
//   warp 26        copy warp of the staged epilogue: one tensor store per half, then -- once the copy has read the half -- the
//                  hand-back to the epilogue, which with a shortcut is the tensor load of the next tile's operand into it.
//
// Tensor memory (512 columns): accumulators 2 x 128, then 16 columns of scale factors (every byte 0x7F = 2^0).
// Every wait on an mbarrier is bounded.  When one runs out, every role leaves its loops, the producer and the copy warp wait
// (bounded) for the copies they still have in flight, the issuer for its MMAs, the tensor memory is released, a status word is
// set, and the kernel returns by itself.
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
constexpr int TP_COPY_WARP = TP_MMA_WARP + 1;
constexpr int TP_THREADS = (TP_COPY_WARP + 1) * 32;
constexpr int TP_RAW_KB = 2;                  // 128-bit pieces per raw stage: 32 bytes = one 256-bit K block per operand row
static_assert(TP_RAW_KB == 2, "the expanders read a row as two 16-byte halves");
constexpr int TP_RAW_STAGES = 6;
constexpr int TP_STAGES = 3;                  // operand stages: the pixel tile and the filter tile of one 256-bit K block, 16 KB each
constexpr int TP_ROWS = TC_PIX + TP_NF;
constexpr int TP_SLOT_BYTES = TP_NF * 128;     // one tile of a stage (128 rows of 128 bytes); TC_PIX == TP_NF
constexpr int TP_STAGE_BYTES = 2 * TP_SLOT_BYTES;
constexpr int TP_RAW_STAGE_BYTES = TP_ROWS * 16 * TP_RAW_KB;
constexpr int TP_RAW_PIX_BYTES = TC_PIX * 16 * TP_RAW_KB;
constexpr int TP_HALF_ROWS = TP_NF / 2;       // filters per half of the staging buffer
constexpr int TP_HALF_BYTES = TP_HALF_ROWS * TC_PIX * 4;
constexpr int TP_OUT_BYTES = 2 * TP_HALF_BYTES;    // one tile of fp32 results [filter][pixel], staged for bulk stores, in two halves
constexpr int TP_SMEM_BYTES = TP_STAGES * TP_STAGE_BYTES + TP_RAW_STAGES * TP_RAW_STAGE_BYTES + TP_OUT_BYTES + 1024;   // + slack to align to 1024
constexpr int TP_TMEM_COLS = 512;
constexpr int TP_SF_COL = 2 * TP_NF;          // scale factors of the pixel operand (4 columns used); the filter operand's at + 8

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

// Tile number -> first filter, first operand row (pixel), and for the staged epilogue the image, the first pixel inside it and
// the number of pixels of the tile that belong to that image.  With the staged epilogue no tile crosses an image (every image
// has its own last, partly used tile: what lies behind it in the operand is computed and dropped), so that a half tile always
// leaves, and its shortcut operand always arrives, as ONE tensor copy; otherwise the tiles run over all pixels of the batch.
struct TileAt
{
	int f0, n0, img, pix0, valid;
};

__device__ __forceinline__ TileAt tile_at(const TcParams & p, int t)
{
	TileAt a;
	const int nt = t / p.tiles_f;
	a.f0 = (t - nt * p.tiles_f) * TP_NF;
	if (p.tiles_per_image > 0)
	{
		a.img = nt / p.tiles_per_image;
		a.pix0 = (nt - a.img * p.tiles_per_image) * TC_PIX;
		a.n0 = a.img * p.n_per_image + a.pix0;
		a.valid = min(TC_PIX, p.n_per_image - a.pix0);
	}
	else
	{
		a.img = 0;
		a.pix0 = 0;
		a.n0 = nt * TC_PIX;
		a.valid = min(TC_PIX, p.n_total - a.n0);
	}
	return a;
}

__global__ void __launch_bounds__(TP_THREADS, 1)
xnor_gemm_tcp_kernel(const TcParams p, const __grid_constant__ CUtensorMap map_pix, const __grid_constant__ CUtensorMap map_fil,
		const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_sc)
{
	constexpr int NF = TP_NF;
	extern __shared__ uint8_t tp_smem_raw[];
	__shared__ uint64_t raw_full[TP_RAW_STAGES];
	__shared__ uint64_t raw_empty[TP_RAW_STAGES];
	__shared__ uint64_t op_full[TP_STAGES];                   // both expanders' arrivals: the stage's pixel and filter bytes are in place
	__shared__ uint64_t op_empty[TP_STAGES];                  // tcgen05.commit: the MMAs that read the stage have completed
	__shared__ uint64_t acc_full[2];
	__shared__ uint64_t acc_empty[2];
	__shared__ uint64_t comb_full[2];
	__shared__ uint64_t out_full[2];                          // per half of the staging buffer: every epilogue warp has staged its part
	__shared__ uint64_t half_ready[2];                        // per half: free for the next tile, and that tile's shortcut operand is in it
	__shared__ uint64_t drain_bar;
	__shared__ uint32_t tmem_base_slot;
	__shared__ __align__(16) int s_fil[2][3][NF];             // per accumulator buffer and filter: unused | mean bits | bias bits
	__shared__ uint32_t raw_seen[TP_THREADS / 32][32];         // written only: see the expanders' release of a raw stage
	__shared__ int s_failed_storage;
	volatile int * s_failed = &s_failed_storage;

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const uint32_t fil_base = (smem_u32(tp_smem_raw) + 1023u) & ~1023u;
	const uint32_t raw_base = fil_base + (uint32_t)(TP_STAGES * TP_STAGE_BYTES);
	const uint32_t out_base = raw_base + (uint32_t)(TP_RAW_STAGES * TP_RAW_STAGE_BYTES);
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
			mbar_init(&comb_full[b], TP_EPI_WARPS);
		}
		for (int h = 0; h < 2; ++h)
		{
			mbar_init(&out_full[h], TP_EPI_WARPS);
			mbar_init(&half_ready[h], 1);
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
	if (warp < 4)
	{
		// the scale factors of both operands: 16 columns of 2^0 on every lane (warps 0..3 sit on the four lane quarters)
		const uint32_t taddr = tmem_base + (uint32_t)TP_SF_COL + ((uint32_t)(warp * 32) << 16);
		asm volatile(
			"tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
			:: "r"(taddr), "r"(0x7F7F7F7Fu) : "memory");
		asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

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
			const TileAt at = tile_at(p, t);
			const int f0 = at.f0;
			const int n0 = at.n0;
			// thread 128 + j of the 256 epilogue threads fetches filter j's constants; the buffer's previous readers are through
			// (every epilogue warp has passed comb_full of the tile in between)
			const bool is_fil = tid >= TC_PIX;
			const int f_row = f0 + tid - TC_PIX;
			if (is_fil)
			{
				const float mean = (f_row < p.M && p.mean_arr != nullptr) ? __ldg(p.mean_arr + f_row) : 0.0f;
				const float bias = (f_row < p.M && p.bias != nullptr) ? __ldg(p.bias + f_row) : 0.0f;
				s_fil[buf][0][tid - TC_PIX] = 0;
				s_fil[buf][1][tid - TC_PIX] = __float_as_int(mean);
				s_fil[buf][2][tid - TC_PIX] = __float_as_int(bias);
			}
			__syncwarp();
			if (lane == 0) { mbar_arrive(&comb_full[buf]); }
			if (!mbar_wait<32>(&comb_full[buf], ph, s_failed, limit)) { break; }
			if (!mbar_wait<512>(&acc_full[buf], ph, s_failed, limit)) { break; }
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			if (!p.bulk_out)
			{
				epilogue_tile<NF, true>(p, nullptr, FilterConsts{&s_fil[buf][0][0], NF}, tmem_base + (uint32_t)(buf * NF), quarter, lane, share,
						TP_EPI_WARPS / 4, f0, n0);
				asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
				__syncwarp();
				if (lane == 0) { mbar_arrive(&acc_empty[buf]); }
				continue;
			}
			// fp32 rows that are contiguous in memory (the layer's output, or the sum with a shortcut operand): the results go to
			// shared memory as [filter][pixel], in two halves of 64 filters, and the copy warp writes each half with one tensor
			// store (a tile never crosses an image in this mode, see tile_at).  Ordinary stores from 8 warps would limit the
			// tile rate: a store is only retired when the L2 has taken it, and in steady state that means evicting a dirty
			// line.  With a shortcut the copy warp has brought the operand into the same place beforehand.
			{
				const int pix_local = quarter * 32 + lane;
				const float pad = (float)p.pad_bits;
				const float slope = p.leaky ? 0.1f : 1.0f;
				const bool has_bias = (p.bias != nullptr);
				const uint32_t tlane = tmem_base + (uint32_t)(buf * NF) + ((uint32_t)(quarter * 32) << 16);
				const bool sc_mode = (p.bulk_out == 2);
				const bool col_ok = pix_local < at.valid;
				const int my_img = at.img;
				const int my_pix = at.pix0 + pix_local;
				uint32_t * sum_words = (sc_mode && p.x.sum_signs != nullptr)
						? p.x.sum_signs + ((size_t)my_img * (p.M >> 5) + (f0 >> 5)) * p.n_per_image + my_pix : nullptr;
				uint32_t * row_words = (sc_mode && p.x.sum_rows != nullptr)
						? p.x.sum_rows + ((size_t)my_img * p.n_per_image + my_pix) * p.x.sum_ldw + (f0 >> 5) : nullptr;
				const bool want_words = (!sc_mode && (p.signs != nullptr || p.x.n_sinks > 0));
				bool alive = true;
				#pragma unroll 1
				for (int half = 0; half < 2; ++half)
				{
					const int chunk = half * 2 + share;           // this warp's 32 filters of the half
					if (f0 + half * TP_HALF_ROWS >= p.M)
					{
						// the half lies behind the last filter: nothing to compute, only the hand-overs (the copy warp skips it too)
						if (half == 1)
						{
							asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
							__syncwarp();
							if (lane == 0) { mbar_arrive(&acc_empty[buf]); }
						}
						__syncwarp();
						if (lane == 0) { mbar_arrive(&out_full[half]); }
						continue;
					}
					uint32_t d[32];
					tmem_load<32>(tlane + (uint32_t)(chunk * 32), d);
					asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
					if (half == 1)
					{
						// the accumulator is read: the issuer may fill it again
						asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
						__syncwarp();
						if (lane == 0) { mbar_arrive(&acc_empty[buf]); }
					}
					// the previous tile's copies have read this half (and this tile's shortcut operand has arrived in it)
					if (!mbar_wait<32>(&half_ready[half], (uint32_t)(it & 1), s_failed, limit)) { alive = false; break; }
					uint32_t word = 0;
					#pragma unroll
					for (int j0 = 0; j0 < 32; j0 += 8)
					{
						// eight filters' constants first (16-byte reads), then the values, then the stores
						int fx[8], fm[8], fb[8];
						FilterConsts{&s_fil[buf][0][0], NF}.load<8>(chunk * 32 + j0, fx, fm, fb);
						float v[8];
						#pragma unroll
						for (int j = 0; j < 8; ++j)
						{
							v[j] = __fmul_rn(__fsub_rn(__uint_as_float(d[j0 + j]), pad), __int_as_float(fm[j]));
							if (has_bias) { v[j] = __fadd_rn(v[j], __int_as_float(fb[j])); }
							v[j] = fmaxf(v[j], __fmul_rn(v[j], slope));
						}
						if (want_words)
						{
							#pragma unroll
							for (int j = 0; j < 8; ++j) { word |= (v[j] > 0.0f ? 1u : 0u) << (j0 + j); }
						}
						if (sc_mode)
						{
							// the sum with the shortcut operand takes the value's place
							float sc[8];
							#pragma unroll
							for (int j = 0; j < 8; ++j)
							{
								asm volatile("ld.shared.f32 %0, [%1];" : "=f"(sc[j]) : "r"(out_base + (uint32_t)(((chunk * 32 + j0 + j) * TC_PIX + pix_local) * 4)));
							}
							#pragma unroll
							for (int j = 0; j < 8; ++j)
							{
								v[j] = __fadd_rn(sc[j], v[j]);
								word |= (v[j] > 0.0f ? 1u : 0u) << (j0 + j);
							}
						}
						#pragma unroll
						for (int j = 0; j < 8; ++j)
						{
							asm volatile("st.shared.f32 [%0], %1;" :: "r"(out_base + (uint32_t)(((chunk * 32 + j0 + j) * TC_PIX + pix_local) * 4)), "f"(v[j]));
						}
					}
					// staged values -> visible to the bulk-copy engine; the copy warp takes the half once every warp's part is in place
					asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
					__syncwarp();
					if (lane == 0) { mbar_arrive(&out_full[half]); }
					if (want_words)
					{
						// the layer's sign words and the consumers' operands behind its sinks (filters past M have value 0: bit clear)
						emit_sign_word(p, word, col_ok && f0 + chunk * 32 < p.M, my_img, my_pix, my_pix, n0 + pix_local, (f0 + chunk * 32) >> 5);
					}
					if (sc_mode && col_ok && f0 + chunk * 32 < p.M)
					{
						// sign words of the sum (32 filters = one channel-packed word of this pixel); filters past M stay clear
						const int left = p.M - (f0 + chunk * 32);
						if (left < 32) { word &= (1u << left) - 1u; }
						if (sum_words != nullptr) { sum_words[(size_t)chunk * p.n_per_image] = word; }
						if (row_words != nullptr) { row_words[chunk] = word; }
					}
				}
				if (!alive) { break; }
			}
		}
	}
	else if (warp == TP_COPY_WARP)
	{
		// ---- copy warp: writes the staged halves, hands them back, and fetches the next tile's shortcut operand ---------
		if (p.bulk_out != 0)
		{
			const bool sc_mode = (p.bulk_out == 2);
			uint32_t requested[2] = {0, 0};                   // completions of half_ready[h] asked for so far
			// Makes half h ready for tile t2: with a shortcut, the copy of its operand (which completes the barrier through its
			// byte count); without, the barrier's one arrival.
			auto request = [&](int t2, int h)
			{
				++requested[h];
				const TileAt at = tile_at(p, t2);
				const int f2 = at.f0 + h * TP_HALF_ROWS;
				if (lane != 0) { return; }
				if (!sc_mode || f2 >= p.M)                    // no operand to fetch, or the half lies behind the last filter
				{
					mbar_arrive(&half_ready[h]);
					return;
				}
				mbar_expect_tx(&half_ready[h], (uint32_t)TP_HALF_BYTES);      // a clipped box still counts in full
				asm volatile(
					"cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
					:: "r"(out_base + (uint32_t)(h * TP_HALF_BYTES)), "l"(reinterpret_cast<uint64_t>(&map_sc)), "r"(at.pix0), "r"(f2), "r"(at.img),
					   "r"(smem_u32(&half_ready[h])) : "memory");
			};
			if ((int)blockIdx.x < p.tiles)
			{
				request(blockIdx.x, 0);
				request(blockIdx.x, 1);
			}
			int it = 0;
			bool ok = true;
			for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it)
			{
				const TileAt at = tile_at(p, t);
				for (int h = 0; h < 2; ++h)
				{
					ok = mbar_wait<64>(&out_full[h], (uint32_t)(it & 1), s_failed, limit);
					if (!ok) { break; }
					const int fh = at.f0 + h * TP_HALF_ROWS;
					if (lane == 0 && fh < p.M)
					{
						// one tensor store per half: filters past M and pixels past the end of the image are clipped
						asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
								:: "l"(reinterpret_cast<uint64_t>(&map_out)), "r"(at.pix0), "r"(fh), "r"(at.img), "r"(out_base + (uint32_t)(h * TP_HALF_BYTES))
								: "memory");
					}
					asm volatile("cp.async.bulk.commit_group;" ::: "memory");
					// once the copies have read the half it belongs to the next tile
					asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
					__syncwarp();
					if (t + (int)gridDim.x < p.tiles) { request(t + (int)gridDim.x, h); }
				}
			}
			// nothing of this CTA may still be in flight when it exits: the stores, and (after a failed wait) requested operands
			asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
			for (int h = 0; h < 2; ++h)
			{
				if (requested[h] > 0) { mbar_wait_plain(&half_ready[h], (requested[h] - 1) & 1u, limit); }
			}
		}
		__syncwarp();
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
				const TileAt at = tile_at(p, t);
				const int f0 = at.f0;
				const int n0 = at.n0;
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
			// instruction descriptor (block-scaled): A = B = e2m1, both K-major, scales ue8m0, N = NF, M = 128, K = 64
			const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(NF >> 3) << 17) | (1u << 23) | ((uint32_t)(TC_PIX >> 4) << 24);
			const uint32_t sfa = tmem_base + (uint32_t)TP_SF_COL;
			const uint32_t sfb = sfa + 8u;
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
				for (int c = 0; c < chunks; ++c, ++sc)
				{
					const uint32_t es = sc % TP_STAGES;
					ok = mbar_wait<0>(&op_full[es], (sc / TP_STAGES) & 1u, s_failed, limit);
					if (!ok) { break; }
					asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
					const uint32_t pix_addr = fil_base + es * (uint32_t)TP_STAGE_BYTES;
					const uint32_t fil_addr = pix_addr + (uint32_t)TP_SLOT_BYTES;
					#pragma unroll
					for (int k = 0; k < 4; ++k)                   // 64 elements = 32 bytes of every row per instruction
					{
						const uint32_t accumulate = (c > 0 || k > 0) ? 1u : 0u;
						asm volatile(
							"{\n\t.reg .pred p;\n\t"
							"setp.ne.b32 p, %4, 0;\n\t"
							"tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
							:: "r"(acc), "l"(make_smem_desc(pix_addr + k * 32)), "l"(make_smem_desc(fil_addr + k * 32)), "r"(idesc),
							   "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
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
		// ---- expanders: pixel rows (warps 8..15) and filter rows (warps 16..23) -> the stage's tiles in shared memory -----------
		const bool is_pix = warp < TP_FIL_WARP0;
		const int grp = ((is_pix ? warp - TP_PIX_WARP0 : warp - TP_FIL_WARP0) >> 2);
		const int row = (warp & 3) * 32 + lane;               // row of the tile this thread owns
		const uint32_t raw_row = raw_base + (uint32_t)((is_pix ? row : TC_PIX + row) * 16 * TP_RAW_KB);
		// this thread's row in stage 0 (pixel tile first, filter tile behind it), swizzle folded in
		const uint32_t row_swz0 = (fil_base + (is_pix ? 0u : (uint32_t)TP_SLOT_BYTES) + (uint32_t)row * 128u) ^ ((uint32_t)(row & 7) << 4);
		const int swap = (lane >> 2) & 1;
		const bool withhold = (p.withhold != 0 && warp == TP_PIX_WARP0);
		uint32_t rc = 0;                                      // raw chunks = operand stages passed so far (every warp counts all of them)
		bool ok = true;
		for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x)
		{
			for (int c = 0; c < chunks && ok; ++c, ++rc)
			{
				if ((int)(rc % TP_GROUPS) != grp) { continue; }              // the other group's chunk
				const uint32_t rs = rc % TP_RAW_STAGES;
				ok = mbar_wait<128>(&raw_full[rs], (rc / TP_RAW_STAGES) & 1u, s_failed, limit);
				if (!ok) { break; }
				// Rows are 32 bytes apart, so the eight lanes of a quarter warp would meet in the same banks twice if each read
				// the first half of its row: lanes 4..7 of every eight take the second half first (swap) and put them back in order.
				uint4 w[TP_RAW_KB];
				#pragma unroll
				for (int j = 0; j < TP_RAW_KB; ++j)
				{
					uint4 v;
					asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
							: "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
							: "r"(raw_row + rs * (uint32_t)TP_RAW_STAGE_BYTES + (uint32_t)((j ^ swap) * 16)) : "memory");
					w[j] = v;
				}
				if (swap != 0)
				{
					const uint4 t0 = w[0];
					w[0] = w[1];
					w[1] = t0;
				}
				// The raw stage can take the next copy once the bits are in registers.  A store of the loaded words comes first: the
				// warp cannot issue it before the loads have returned, and the arrival follows it in program order.  Without it the
				// arrival could be performed while the loads still waited in the shared-memory pipeline (seen under heavy
				// shared-memory traffic: the next copy overwrote the first pixel rows of the stage before they were read).
				{
					uint32_t got = 0;
					#pragma unroll
					for (int j = 0; j < TP_RAW_KB; ++j) { got |= w[j].x | w[j].y | w[j].z | w[j].w; }
					asm volatile("st.shared.b32 [%0], %1;" :: "r"(smem_u32(&raw_seen[warp][lane])), "r"(got) : "memory");
					__syncwarp();
					if (lane == 0) { mbar_arrive(&raw_empty[rs]); }
				}
				const uint32_t es = rc % TP_STAGES;
				if (rc >= (uint32_t)TP_STAGES)
				{
					// the MMAs that read this stage (issued TP_STAGES stages ago) must have completed
					ok = mbar_wait<128>(&op_empty[es], (rc / TP_STAGES - 1) & 1u, s_failed, limit);
					if (!ok) { break; }
				}
				expand_row_fp4(row_swz0 + es * (uint32_t)TP_STAGE_BYTES, w[0], w[1]);
				// generic-proxy writes -> visible to the tensor core's async proxy
				asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
				__syncwarp();
				if (lane == 0 && !(withhold && rc == 0)) { mbar_arrive(&op_full[es]); }
			}
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

// Tensor map of an fp32 tensor [images][M][ldc] (the output, or a shortcut operand) for boxes of 128 pixels x 64 filters of one image.
static int make_out_map(CUtensorMap * map, float * base, int n_per_image, int M, int images, int ldc)
{
	EncodeTiledFn enc = tensor_map_encoder();
	if (enc == nullptr) { return XNOR_B200_ERR_CUDA; }
	const cuuint64_t dims[3] = {(cuuint64_t)n_per_image, (cuuint64_t)M, (cuuint64_t)images};
	const cuuint64_t strides[2] = {(cuuint64_t)ldc * 4, (cuuint64_t)M * (cuuint64_t)ldc * 4};
	const cuuint32_t box[3] = {(cuuint32_t)TC_PIX, (cuuint32_t)TP_HALF_ROWS, 1};
	const cuuint32_t elem[3] = {1, 1, 1};
	const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, elem,
			CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS)
	{
		g_last_cuda_error = (int)cudaErrorInvalidValue;
		return XNOR_B200_ERR_CUDA;
	}
	return XNOR_B200_OK;
}

// What the staged epilogue can write: fp32 rows that are contiguous runs of whole 16-byte pieces, in plain pixel order, with sign
// words beside them.  1: the layer's own output (+ its sign words and sinks); 2: only the sum with a shortcut operand of the
// same layout (+ the sum's sign words); 0: neither.
int tcp_stages_output(const TcParams & p)
{
	if (p.counts != nullptr || p.x.win_w != 0) { return 0; }
	// images smaller than a tile would leave most of every tile idle (and the tensor maps' boxes wider than the tensor)
	if (p.n_per_image < TC_PIX || p.n_per_image % 4 != 0 || p.n_total % p.n_per_image != 0 || p.ldc % 4 != 0) { return 0; }
	if (p.shortcut_in == nullptr)
	{
		// the layer's sign words and plain (or upsampling) sinks ride along: one word per pixel and 32 filters
		return (p.C != nullptr && p.x.sum_signs == nullptr && p.x.sum_rows == nullptr && (((uintptr_t)p.C) & 15u) == 0) ? 1 : 0;
	}
	if (p.signs != nullptr || p.x.n_sinks != 0) { return 0; }
	return (p.C == nullptr && p.shortcut_out != nullptr && ((((uintptr_t)p.shortcut_in) | ((uintptr_t)p.shortcut_out)) & 15u) == 0) ? 2 : 0;
}

static int launch_tcp(TcParams & p, cudaStream_t stream)
{
	p.tiles_f = (p.M + TP_NF - 1) / TP_NF;
	p.bulk_out = tcp_stages_output(p);
	// staged epilogue: tiles per image (none crosses an image); otherwise tiles over all pixels of the batch
	p.tiles_per_image = (p.bulk_out != 0) ? (p.n_per_image + TC_PIX - 1) / TC_PIX : 0;
	const long long tiles_n = (p.bulk_out != 0) ? (long long)p.tiles_per_image * (p.n_total / p.n_per_image) : (p.n_total + TC_PIX - 1) / TC_PIX;
	const long long tiles = (long long)p.tiles_f * tiles_n;
	if (tiles > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	p.tiles = (int)tiles;
	// 256-bit K blocks; what they cover behind K is zero in both operands (rows are zero-padded, the copies zero-fill)
	p.pad_bits = ((p.kblocks + TP_RAW_KB - 1) / TP_RAW_KB) * 256 - p.K;
	CUtensorMap map_pix, map_fil;
	int rc = make_row_map(&map_pix, p.B, p.n_total, (size_t)p.ldb_words * 4, TC_PIX);
	if (rc != XNOR_B200_OK) { return rc; }
	rc = make_row_map(&map_fil, p.A, p.M, (size_t)p.lda_words * 4, TP_NF);
	if (rc != XNOR_B200_OK) { return rc; }
	CUtensorMap map_out = map_fil, map_sc = map_fil;          // valid maps in any case; only read when bulk_out is set
	if (p.bulk_out != 0)
	{
		rc = make_out_map(&map_out, (p.bulk_out == 2) ? p.shortcut_out : p.C, p.n_per_image, p.M, p.n_total / p.n_per_image, p.ldc);
		if (rc != XNOR_B200_OK) { return rc; }
	}
	if (p.bulk_out == 2)
	{
		rc = make_out_map(&map_sc, const_cast<float *>(p.shortcut_in), p.n_per_image, p.M, p.n_total / p.n_per_image, p.ldc);
		if (rc != XNOR_B200_OK) { return rc; }
	}
	rc = ensure_dynamic_smem((const void *)xnor_gemm_tcp_kernel, TP_SMEM_BYTES);
	if (rc != XNOR_B200_OK) { return rc; }
	const int grid = (int)((tiles < (long long)sm_count()) ? tiles : (long long)sm_count());
	xnor_gemm_tcp_kernel<<<grid, TP_THREADS, TP_SMEM_BYTES, stream>>>(p, map_pix, map_fil, map_out, map_sc);
	return check_launch();
}

int launch_xnor_gemm_tcp(TcParams & p, cudaStream_t stream)
{
	return launch_tcp(p, stream);
}

}  // namespace xnor
