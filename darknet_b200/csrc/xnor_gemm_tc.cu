// XNOR GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for large layers.
//
// tcgen05.mma has no 1-bit operand kind, and the legacy mma.sync b1 path measures slower than the integer pipe on this GPU.
// A binary dot product is nevertheless an ordinary GEMM once a set bit is read as +1 and a clear bit as -1:
//     D[j][i] = sum_k b_jk * a_ik = (agreeing positions) - (disagreeing positions) = 2 * agreeing - K
// The narrowest operand type the tensor core takes is the 4-bit float e2m1 (kind::mxf4, block-scaled, K = 64 per instruction,
// twice the rate of the 8-bit kinds): +1.0 is 0x2, -1.0 is 0xA, both scale-factor operands are held at 2^0, and the fp32
// accumulator adds integers of magnitude <= K exactly.  The packed operands stay 1 bit per element in HBM and L2 (the same
// buffers the integer-pipe kernel reads) and are widened to 4 bits only inside shared memory, next to the tensor core that
// consumes them.  Positions behind K that a K block covers are zero bits in both rows, i.e. (-1)(-1) = +1 each: the epilogue
// subtracts their number (TcParams::pad_bits).
//
// Orientation: the UMMA "M" dimension (128 TMEM lanes) carries OUTPUT PIXELS, the "N" dimension (TMEM columns)
// carries FILTERS.  After tcgen05.ld each thread then owns one pixel and 32 consecutive filters per load, so
// for every filter the 32 lanes of a warp store 32 consecutive pixels: NCHW output rows are written with fully
// coalesced 128-byte stores.
//
// One CTA = 128 pixels x NF filters (NF = 32, 64 or 128), warp-specialised:
//   warp 0            allocates TMEM (NF accumulator columns + 16 columns of scale factors, rounded to a power of two); one
//                     lane issues, per 256-bit K block, 4 x tcgen05.mma.cta_group::1.kind::mxf4.block_scale (M=128, N=NF,
//                     K=64) and a tcgen05.commit that frees the stage when the MMAs have read it;
//   warps 1..(128+NF)/32   producers: each thread owns one operand row (pixel row or filter row), keeps two
//                     K blocks of packed bits in flight from L2, expands 256 bits -> 128 bytes straight into the
//                     canonical K-major SWIZZLE_128B tile of the current stage, and its warp arrives on the stage's
//                     "full" barrier; warps 1..4 first write the scale factors; the same warps run the epilogue.
// Two or three stages per CTA and two to four CTAs per SM (tensor memory allows 512 columns per SM): while one CTA drains
// its accumulators the others keep the tensor core busy.  The epilogue applies mean scale, bias and leaky with the same
// two-rounding fp32 sequence as the integer-pipe kernel, so both kernels give bit-identical outputs.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in g_tc_error, all roles drop out
// of their loops, the TMEM columns are still released, and the kernel returns.
#include "tc_common.cuh"

#include <mutex>
namespace xnor
{

// Sticky status word: set to 1 by a tensor-core GEMM kernel (either of the two) whose bounded wait ran out.
__device__ int g_tc_error = 0;

int tc_fill_launch_fields(TcParams & p)
{
	constexpr int MAX_DEVICES = 64;
	static std::mutex mu;
	static int * ptrs[MAX_DEVICES] = {nullptr};
	int dev = 0;
	cudaError_t e = cudaGetDevice(&dev);
	if (e != cudaSuccess) { return cuda_fail(e); }
	if (dev < 0 || dev >= MAX_DEVICES) { return XNOR_B200_ERR_INVALID; }
	{
		std::lock_guard<std::mutex> lock(mu);
		if (ptrs[dev] == nullptr)
		{
			void * sym = nullptr;
			e = cudaGetSymbolAddress(&sym, g_tc_error);
			if (e != cudaSuccess) { return cuda_fail(e); }
			ptrs[dev] = (int *)sym;
		}
		p.status = ptrs[dev];
	}
	p.spin_limit = (tuning().tc_wait_polls > 0) ? (uint32_t)tuning().tc_wait_polls : TC_SPIN_LIMIT;
	p.withhold = tuning().tc_withhold_arrival;
	return XNOR_B200_OK;
}

template <int NF>
struct TcShape
{
	static constexpr int ROWS = TC_PIX + NF;                     // operand rows per stage
	static constexpr int PRODUCER_WARPS = ROWS / 32;
	static constexpr int THREADS = 32 + ROWS;                    // warp 0 + producers
	static constexpr int STAGES = (NF == 128) ? 3 : 2;
	static constexpr int PIX_TILE_BYTES = TC_PIX * 128;
	static constexpr int STAGE_BYTES = ROWS * 128;               // one 256-bit K block of every row, four bits per element
	static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;   // + slack to align the ring to 1024 bytes
	// tensor memory: NF accumulator columns, then 16 columns of scale factors (every byte 0x7F = 2^0); a power of two
	static constexpr int TMEM_COLS = (NF <= 32) ? 64 : (NF <= 64) ? 128 : 256;
	static constexpr int SF_COL = NF;                            // scale factors of the pixel operand: 4 columns
	static constexpr int SFB_COL = NF + 8;                       // scale factors of the filter operand: NF / 32 columns
	static constexpr int CTAS_PER_SM = (NF == 128) ? 2 : 4;      // tensor-memory columns and shared memory both allow this many
};

template <int NF>
__global__ void __launch_bounds__(TcShape<NF>::THREADS, TcShape<NF>::CTAS_PER_SM)      // co-resident CTAs: one epilogue overlaps another main loop
xnor_gemm_tc_kernel(const TcParams p)
{
	using S = TcShape<NF>;
	constexpr int STAGES = S::STAGES;
	extern __shared__ uint8_t tc_smem_raw[];
	__shared__ uint64_t bar_full[STAGES];
	__shared__ uint64_t bar_empty[STAGES];
	__shared__ uint64_t bar_done;
	__shared__ uint32_t tmem_base_slot;
	__shared__ __align__(16) int s_fil[3][NF];               // per filter: unused | mean bits | bias bits
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
		for (int s = 0; s < STAGES; ++s)
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
				:: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
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
			// instruction descriptor (block-scaled): A = B = e2m1, both K-major, scales ue8m0, N = NF, M = 128, K = 64
			const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(NF >> 3) << 17) | (1u << 23) | ((uint32_t)(TC_PIX >> 4) << 24);
			const uint32_t sfa = tmem_base + (uint32_t)S::SF_COL;
			const uint32_t sfb = tmem_base + (uint32_t)S::SFB_COL;
			bool ok = true;
			for (int kb = 0; kb < p.kblocks && ok; ++kb)
			{
				const int s = kb % STAGES;
				ok = mbar_wait(&bar_full[s], (uint32_t)((kb / STAGES) & 1), s_failed, p.spin_limit);
				if (!ok) { break; }
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t pix_addr = ring + (uint32_t)s * S::STAGE_BYTES;
				const uint32_t fil_addr = pix_addr + S::PIX_TILE_BYTES;
				#pragma unroll
				for (int k = 0; k < 4; ++k)                       // 64 elements = 32 bytes of every row per instruction
				{
					const uint64_t adesc = make_smem_desc(pix_addr + k * 32);
					const uint64_t bdesc = make_smem_desc(fil_addr + k * 32);
					const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
					asm volatile(
						"{\n\t.reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
						:: "r"(tmem_base), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
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
		if (warp <= 4)
		{
			// the scale factors of both operands: 16 columns of 2^0 on every lane (warps 1..4 sit on the four lane quarters);
			// ordered before the first MMA by this warp's first arrival on bar_full
			const uint32_t taddr = tmem_base + (uint32_t)S::SF_COL + ((uint32_t)((warp & 3) * 32) << 16);
			const uint32_t one = 0x7F7F7F7Fu;
			asm volatile(
				"tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
				:: "r"(taddr), "r"(one) : "memory");
			asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
		}
		const int r = tid - 32;                               // operand row of this thread within the stage
		const bool is_pix = r < TC_PIX;
		const int row_in_tile = is_pix ? r : r - TC_PIX;
		const bool row_ok = is_pix ? (n0 + row_in_tile < p.n_total) : (f0 + row_in_tile < p.M);
		const int ld_words = is_pix ? p.ldb_words : p.lda_words;
		const int ld4 = ld_words >> 2;                        // 16-byte pieces of the row that exist
		const uint4 * src = reinterpret_cast<const uint4 *>(
				is_pix ? p.B + (size_t)(row_ok ? n0 + row_in_tile : 0) * p.ldb_words
				       : p.A + (size_t)(row_ok ? f0 + row_in_tile : 0) * p.lda_words);
		// byte address of this thread's row in stage 0, swizzle term folded in
		const uint32_t row_swz0 = (ring + (is_pix ? 0u : (uint32_t)S::PIX_TILE_BYTES) + (uint32_t)row_in_tile * 128u)
				^ ((uint32_t)(row_in_tile & 7) << 4);
		const uint4 zero4 = make_uint4(0, 0, 0, 0);
		// piece i of the row, zero behind the end of the row (rows are a multiple of 128 bits long, K blocks of 256)
		auto piece = [&](int i) { return (row_ok && i < ld4 && i < 2 * p.kblocks) ? __ldg(src + i) : zero4; };
		uint4 a0 = piece(0), a1 = piece(1), b0 = piece(2), b1 = piece(3);
		bool ok = true;
		for (int kb = 0; kb < p.kblocks; ++kb)
		{
			const int s = kb % STAGES;
			const uint4 lo = a0, hi = a1;
			a0 = b0; a1 = b1;
			b0 = piece(2 * kb + 4); b1 = piece(2 * kb + 5);
			if (kb >= STAGES)
			{
				// the MMAs that read this stage (issued STAGES blocks ago) must have completed
				ok = mbar_wait(&bar_empty[s], (uint32_t)((kb / STAGES - 1) & 1), s_failed, p.spin_limit);
				if (!ok) { break; }
			}
			expand_row_fp4(row_swz0 + (uint32_t)s * S::STAGE_BYTES, lo, hi);
			// generic-proxy writes -> visible to the tensor core's async proxy; then one arrival per warp
			asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
			__syncwarp();
			if (lane == 0 && !(p.withhold != 0 && kb == 0 && warp == 1)) { mbar_arrive(&bar_full[s]); }
		}
		if (!is_pix)
		{
			const int f = f0 + row_in_tile;
			const float mean = (f < p.M && p.mean_arr != nullptr) ? __ldg(p.mean_arr + f) : 0.0f;
			const float bias = (f < p.M && p.bias != nullptr) ? __ldg(p.bias + f) : 0.0f;
			s_fil[0][row_in_tile] = 0;
			s_fil[1][row_in_tile] = __float_as_int(mean);
			s_fil[2][row_in_tile] = __float_as_int(bias);
		}
	}

	// ---- the accumulators are complete when the issuing thread has seen bar_done; everyone else meets it at the barrier ----
	if (tid == 0) { mbar_wait<64>(&bar_done, 0, s_failed, p.spin_limit); }
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const bool failed = (*s_failed != 0);

	if (!failed && warp != 0)
	{
		// the producer warps 1..PRODUCER_WARPS cover every TMEM lane quarter PRODUCER_WARPS/4 times; the odd producer warps
		// of the narrow tiles (5 or 6 producer warps) have nothing left to read
		constexpr int SHARES = S::PRODUCER_WARPS / 4;
		const int share = ((warp - 1) >> 2) < SHARES ? ((warp - 1) >> 2) : NF;
		epilogue_tile<NF, true>(p, nullptr, FilterConsts{&s_fil[0][0], NF}, tmem_base, warp & 3, lane, share, SHARES, f0, n0);
	}
	else if (failed && tid == 0)
	{
		atomicExch(p.status, 1);
	}

	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 0)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
	}
}

bool tc_gemm_eligible(int M, int n_total, int K)
{
	// The faster of two estimates fitted to measurements on B200 (batch 8..64 layer shapes) decides:
	//   tensor-core kernel: ~7 us of fixed cost (launch with ~100 KB of shared memory, TMEM allocation, pipeline fill, drain)
	//                       + per tile 0.6 us per 256-bit K block and 2.8 us of start-up and epilogue for 128-filter tiles
	//                       (0.35 + 1.6 and 0.3 + 1.1 for 64 and 32 filters), times the tiles per SM (co-resident CTAs share
	//                       the SM's issue slots and shared-memory bandwidth);
	//   integer kernel:     ~4 us + binary ops (over the K words it actually walks) at 250 T/s + 2 us per million outputs
	//                       (index arithmetic and stores of its epilogue, which dominate when K is short: 1x1 layers
	//                       over 64..256 channels at large batch run 1.3-2x faster on the tensor-core kernel).
	if (M < 16 || K < 64) { return false; }
	const int nf = (M > 64) ? 128 : (M > 32) ? 64 : 32;
	const long long tiles = (long long)((M + nf - 1) / nf) * ((n_total + TC_PIX - 1) / TC_PIX);
	const double kb = (double)((K + 255) / 256);
	const double per_tile = (nf == 128) ? 0.6 * kb + 2.8 : (nf == 64) ? 0.35 * kb + 1.6 : 0.3 * kb + 1.1;
	double load = (double)tiles / (double)sm_count();
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
	p.pad_bits = 0;
	p.C = C; p.ldc = ldc; p.mean_arr = mean_arr; p.bias = bias; p.leaky = leaky;
	p.shortcut_in = shortcut_in; p.shortcut_out = shortcut_out; p.counts = counts;
	int rc = tc_fill_launch_fields(p);
	if (rc != XNOR_B200_OK) { return rc; }
	// The persistent kernel where it measured faster (B200, layer shapes of batch 16..64; us per call, persistent vs one tile per
	// CTA).  fp32-only epilogues, which it writes with tensor stores from shared memory -- plain output: 55.8 vs 87.2 for
	// 512 x 43264 x 2304, 324 vs 424 at 1024 x 43264 x 9216, 46.9 vs 74.2 at 256 x 100352 x 1152, 73.5 vs 108 at
	// 128 x 401408 x 576, 23.1 vs 33.7 at 255 x 43264 x 1024; only the sum with a shortcut operand (darknet53 at batch 32):
	// 58 vs 93 for 256 filters at 56 x 56, 48 vs 62 for 512 at 28 x 28, 285 vs 392 for 64 filters at 224 x 224 (half of each
	// 128-filter tile is idle there, but the layer is bound by its epilogue and its 0.8 GB of fp32 traffic).  Sign words and sinks: from K = 2048
	// on, where its main loop hides the 8 epilogue warps.  An output AND a shortcut sum, or counts, stay with the other kernel.
	// xnor_b200_set_tuning pins either.
#ifndef XNOR_TCP_MIN_K_STAGED
#define XNOR_TCP_MIN_K_STAGED 256
#endif
#ifndef XNOR_TCP_MIN_K_OTHER
#define XNOR_TCP_MIN_K_OTHER 2048
#endif
	const int variant = tuning().tc_kernel;
	const int staged = tcp_stages_output(p);
#ifndef XNOR_TCP_MIN_M_STAGED
#define XNOR_TCP_MIN_M_STAGED 33
#endif
	// up to 64 filters half of every 128-filter tile is idle: only worth it where the epilogue is heavy (a shortcut operand to
	// fetch, or sign words / sinks beside the tensor); the plain output of such a layer is 10-15 % faster on the other kernel
	const bool heavy = (staged == 2 || (staged == 1 && (signs != nullptr || p.x.n_sinks > 0)));
	const bool tcp_can = (M >= (heavy ? XNOR_TCP_MIN_M_STAGED : 65) && counts == nullptr && (shortcut_in == nullptr || staged == 2));
	const bool tcp_wins = tcp_can && K >= (staged != 0 ? XNOR_TCP_MIN_K_STAGED : XNOR_TCP_MIN_K_OTHER);
	if (variant == 2 || (variant == 0 && tcp_wins)) { return launch_xnor_gemm_tcp(p, stream); }
	// the kind::mxf4 kernel walks 256-bit K blocks; what they cover behind K is zero in both operands
	p.kblocks = (K + 255) / 256;
	p.pad_bits = p.kblocks * 256 - K;
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
