// XNOR GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for large layers.
//
// tcgen05.mma has no 1-bit operand kind, and the legacy mma.sync b1 path measures slower than the integer
// pipe on this GPU.  A binary dot product is nevertheless an integer GEMM: with both operands expanded to
// bytes holding 0 or 1,
//     D[i][j] = sum_k a_ik * b_jk = popc(A_i & B_j)            (kind::i8, u8 x u8 -> s32, exact)
//     agreeing bits = K - popc(A_i) - popc(B_j) + 2 * D[i][j]
// so the packed operands stay 1 bit per element in HBM and L2 (same buffers as the integer-pipe kernel) and
// are widened to bytes only inside shared memory, by the same threads that feed the tensor core:
//
//   per 128-bit K block and stage:
//     256 threads: thread t < 128 expands A row t, thread t >= 128 expands B row t-128 (16 bytes of bits ->
//                  128 bytes of 0/1) straight into the canonical K-major SWIZZLE_128B tile layout, and keeps a
//                  running popcount of its row;
//     one thread:  4 x tcgen05.mma.cta_group::1.kind::i8 (M=128, N=128, K=32) accumulating into TMEM, then
//                  tcgen05.commit onto the stage's mbarrier so the stage can be refilled.
//   The MMAs of block k run while the threads expand block k+1; two CTAs fit on one SM and overlap further.
//   Epilogue: tcgen05.ld brings the s32 accumulators back (one TMEM lane = one output row per thread), the
//   popcount correction, mean scale, bias and leaky are applied with the same two-rounding fp32 sequence as the
//   integer-pipe kernel, so both kernels give bit-identical outputs.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in g_tc_error, skips the remaining
// work, still releases its TMEM columns and returns.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int TC_BM = 128;
constexpr int TC_BN = 128;
constexpr int TC_THREADS = 256;
constexpr int TC_STAGES = 3;
constexpr int TC_TILE_BYTES = 128 * 128;                 // one operand tile of one stage: 128 rows x 128 bytes
constexpr int TC_STAGE_BYTES = 2 * TC_TILE_BYTES;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024;   // + slack to align the ring to 1024 bytes
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

__device__ int g_tc_error = 0;

struct TcParams
{
	const uint32_t * A;
	const uint32_t * B;
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
	int tiles_m;
};

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}

// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity)
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
	}
	return false;
}

// 16 bits -> 16 bytes of 0/1 (bit j -> byte j).  (x & 15) * 0x204081 puts bit j of the nibble at bit 8j.
__device__ __forceinline__ uint4 expand16(uint32_t bits)
{
	uint4 v;
	v.x = ((bits & 15u) * 0x204081u) & 0x01010101u;
	v.y = (((bits >> 4) & 15u) * 0x204081u) & 0x01010101u;
	v.z = (((bits >> 8) & 15u) * 0x204081u) & 0x01010101u;
	v.w = (((bits >> 12) & 15u) * 0x204081u) & 0x01010101u;
	return v;
}

// One row of one K block: 128 bits -> 128 bytes at row r of a 128-row K-major tile with the 128-byte swizzle
// (16-byte chunk c of row r is stored at chunk position c ^ (r % 8); tile base 1024-byte aligned).
__device__ __forceinline__ void expand_row(uint32_t tile_addr, int r, const uint4 w)
{
	const uint32_t row = tile_addr + (uint32_t)r * 128u;
	const uint32_t sw = (uint32_t)(r & 7);
	const uint32_t words[4] = {w.x, w.y, w.z, w.w};
	#pragma unroll
	for (int c = 0; c < 8; ++c)
	{
		const uint4 v = expand16(words[c >> 1] >> ((c & 1) * 16));
		asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
				:: "r"(row + (((uint32_t)c ^ sw) << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
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

__global__ void __launch_bounds__(TC_THREADS)
xnor_gemm_tc_kernel(const TcParams p)
{
	extern __shared__ uint8_t tc_smem_raw[];
	__shared__ uint64_t bar_empty[TC_STAGES];
	__shared__ uint64_t bar_done;
	__shared__ uint32_t tmem_base_slot;
	__shared__ int s_pop[TC_BM + TC_BN];
	__shared__ int s_failed;

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const uint32_t ring = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;

	const int tile_m = blockIdx.x % p.tiles_m;
	const int tile_n = blockIdx.x / p.tiles_m;
	const int m0 = tile_m * TC_BM;
	const int n0 = tile_n * TC_BN;

	if (tid == 0)
	{
		for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&bar_empty[s], 1); }
		mbar_init(&bar_done, 1);
		s_failed = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)TC_BN) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = tmem_base_slot;

	// this thread's operand row
	const bool is_a = tid < TC_BM;
	const int r = is_a ? tid : tid - TC_BM;
	const bool row_ok = is_a ? (m0 + r < p.M) : (n0 + r < p.n_total);
	const uint32_t * src = is_a ? p.A + (size_t)(row_ok ? m0 + r : 0) * p.lda_words
	                            : p.B + (size_t)(row_ok ? n0 + r : 0) * p.ldb_words;
	int pop = 0;

	// instruction descriptor: D = s32, A = B = u8, both K-major, N = 128, M = 128
	const uint32_t idesc = (2u << 4) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

	uint4 next = make_uint4(0, 0, 0, 0);
	if (row_ok && p.kblocks > 0) { next = __ldg(reinterpret_cast<const uint4 *>(src)); }
	bool failed = false;

	for (int kb = 0; kb < p.kblocks; ++kb)
	{
		const int s = kb % TC_STAGES;
		const uint4 cur = next;
		if (row_ok && kb + 1 < p.kblocks) { next = __ldg(reinterpret_cast<const uint4 *>(src) + kb + 1); }
		if (kb >= TC_STAGES && !failed)
		{
			// the MMAs that read this stage (issued STAGES blocks ago) must have completed
			if (!mbar_wait(&bar_empty[s], (uint32_t)((kb / TC_STAGES - 1) & 1))) { failed = true; s_failed = 1; }
		}
		if (!failed)
		{
			expand_row(ring + (uint32_t)s * TC_STAGE_BYTES + (is_a ? 0u : (uint32_t)TC_TILE_BYTES), r, cur);
			pop += __popc(cur.x) + __popc(cur.y) + __popc(cur.z) + __popc(cur.w);
		}
		// generic-proxy writes -> visible to the tensor core's async proxy, then hand over to the issuing thread
		asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
		asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
		__syncthreads();
		failed = failed || (s_failed != 0);
		if (tid == 0 && !failed)
		{
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
			const uint32_t a_addr = ring + (uint32_t)s * TC_STAGE_BYTES;
			const uint32_t b_addr = a_addr + TC_TILE_BYTES;
			#pragma unroll
			for (int k = 0; k < 4; ++k)
			{
				const uint64_t adesc = make_smem_desc(a_addr + k * 32);
				const uint64_t bdesc = make_smem_desc(b_addr + k * 32);
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
	}

	if (tid == 0 && !failed)
	{
		asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
				:: "r"(smem_u32(&bar_done)) : "memory");
	}
	s_pop[tid] = pop;
	if (!failed && !mbar_wait(&bar_done, 0)) { failed = true; s_failed = 1; }
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	failed = failed || (s_failed != 0);

	if (!failed)
	{
		// Warp w may read TMEM lanes 32*(w%4) .. +31; warps 0-3 take columns 0-63, warps 4-7 columns 64-127.
		const int lane_base = 32 * (warp & 3);
		const int row_local = lane_base + lane;
		const int m = m0 + row_local;
		const int pop_a = s_pop[row_local];
		const float mean = (m < p.M && p.mean_arr != nullptr) ? __ldg(p.mean_arr + m) : 0.0f;
		const float bias = (m < p.M && p.bias != nullptr) ? __ldg(p.bias + m) : 0.0f;
		#pragma unroll 1
		for (int chunk = 0; chunk < 2; ++chunk)
		{
			const int col0 = (warp >> 2) * 64 + chunk * 32;
			uint32_t d[32];
			const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)col0;
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
			if (m < p.M)
			{
				int col = n0 + col0;
				int img = col / p.n_per_image;
				int pix = col - img * p.n_per_image;
				#pragma unroll
				for (int j = 0; j < 32; ++j, ++col)
				{
					if (col < p.n_total)
					{
						// agreeing bits among the first K
						const int count = p.K - pop_a - s_pop[TC_BM + col0 + j] + 2 * (int)d[j];
						if (p.counts != nullptr)
						{
							p.counts[(size_t)m * p.n_total + col] = count;
						}
						else
						{
							const size_t idx = ((size_t)img * p.M + m) * p.ldc + pix;
							float v = __fmul_rn((float)(2 * count - p.K), mean);
							if (p.bias != nullptr) { v = __fadd_rn(v, bias); }
							if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
							p.C[idx] = v;
							if (p.shortcut_out != nullptr) { p.shortcut_out[idx] = __fadd_rn(__ldg(p.shortcut_in + idx), v); }
						}
					}
					if (++pix == p.n_per_image) { pix = 0; ++img; }
				}
			}
		}
	}
	else if (tid == 0)
	{
		atomicExch(&g_tc_error, 1);
	}

	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 0)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TC_BN) : "memory");
	}
}

bool tc_gemm_eligible(int M, int n_total, int K)
{
	// Needs full 128-row tiles to pay off, enough K to amortise the TMEM round trip, and at least about one
	// tile per SM; everything else stays on the integer-pipe kernel.
	if (M < 96 || K < 512) { return false; }
	const long long tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((n_total + TC_BN - 1) / TC_BN);
	return tiles >= sm_count();
}

int launch_xnor_gemm_tc(int M, int n_total, int n_per_image, int K,
		const uint32_t * A, int lda_words, const uint32_t * B, int ldb_words,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky,
		const float * shortcut_in, float * shortcut_out, int32_t * counts, cudaStream_t stream)
{
	TcParams p;
	p.A = A; p.B = B;
	p.M = M; p.n_total = n_total; p.n_per_image = n_per_image; p.K = K;
	p.lda_words = lda_words; p.ldb_words = ldb_words;
	p.kblocks = (K + 127) / 128;
	p.C = C; p.ldc = ldc; p.mean_arr = mean_arr; p.bias = bias; p.leaky = leaky;
	p.shortcut_in = shortcut_in; p.shortcut_out = shortcut_out; p.counts = counts;
	p.tiles_m = (M + TC_BM - 1) / TC_BM;
	const long long grid = (long long)p.tiles_m * ((n_total + TC_BN - 1) / TC_BN);
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	int rc = ensure_dynamic_smem((const void *)xnor_gemm_tc_kernel, TC_SMEM_BYTES);
	if (rc != XNOR_B200_OK) { return rc; }
	xnor_gemm_tc_kernel<<<(unsigned)grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(p);
	return check_launch();
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
