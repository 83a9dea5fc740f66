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
#include "tc_common.cuh"

#include <mutex>
namespace xnor
{

constexpr int TC_STAGES = 2;

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
	__shared__ __align__(16) int s_fil[3][NF];               // per filter: -2 popc(row) | mean bits | bias bits
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
				ok = mbar_wait(&bar_full[s], (uint32_t)((kb / TC_STAGES) & 1), s_failed, p.spin_limit);
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
				ok = mbar_wait(&bar_empty[s], (uint32_t)((kb / TC_STAGES - 1) & 1), s_failed, p.spin_limit);
				if (!ok) { break; }
			}
			expand_row(row_swz0 + (uint32_t)s * S::STAGE_BYTES, cur);
			pop += __popc(cur.x) + __popc(cur.y) + __popc(cur.z) + __popc(cur.w);
			// generic-proxy writes -> visible to the tensor core's async proxy; then one arrival per warp
			asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
			__syncwarp();
			if (lane == 0 && !(p.withhold != 0 && kb == 0 && warp == 1)) { mbar_arrive(&bar_full[s]); }
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
			s_fil[0][row_in_tile] = -2 * pop;
			s_fil[1][row_in_tile] = __float_as_int(mean);
			s_fil[2][row_in_tile] = __float_as_int(bias);
		}
	}

	// ---- everyone: wait for the accumulators ----------------------------------------------------------
	mbar_wait(&bar_done, 0, s_failed, p.spin_limit);
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
		epilogue_tile<NF>(p, s_pop, FilterConsts{&s_fil[0][0], NF}, tmem_base, warp & 3, lane, share, SHARES, f0, n0);
	}
	else if (failed && tid == 0)
	{
		atomicExch(p.status, 1);
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
	int rc = tc_fill_launch_fields(p);
	if (rc != XNOR_B200_OK) { return rc; }
	// the persistent kernel where it measured faster, unless xnor_b200_set_tuning pinned one of the two
	const int variant = tuning().tc_kernel;
	if (variant == 2 || (variant == 0 && tcp_takes(p))) { return launch_xnor_gemm_tcp(p, stream); }
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
