// Measured ceilings of the tensor-core route of the XNOR GEMM: back-to-back tcgen05.mma from resident shared-memory tiles
// on every SM, no operand traffic and no epilogue -- kind::i8 (M=128, N=256, K=32; the persistent kernel's instruction) and
// kind::mxf4 (M=128, N=256, K=64; the one-tile kernel's).  A GEMM can at best reach its figure; the gap to it is the cost
// of widening bits in shared memory.  Counted like the GEMM itself: 2*M*N*K operations per MMA.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int UP_THREADS = 128;
constexpr int UP_N = 256;
constexpr int UP_SMEM = (128 + UP_N) * 128 + 1024;
constexpr uint32_t UP_SPIN_LIMIT = 1u << 24;

__global__ void __launch_bounds__(UP_THREADS)
umma_i8_peak_kernel(int iters, int * timeouts)
{
	extern __shared__ uint8_t up_smem_raw[];
	__shared__ uint64_t bar;
	__shared__ uint32_t tmem_slot;
	const uint32_t base = ((uint32_t)__cvta_generic_to_shared(up_smem_raw) + 1023u) & ~1023u;
	const uint32_t bar_addr = (uint32_t)__cvta_generic_to_shared(&bar);
	const int warp = threadIdx.x >> 5;

	for (int i = threadIdx.x; i < (128 + UP_N) * 128 / 16; i += UP_THREADS)
	{
		asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" :: "r"(base + i * 16), "r"(0x01000100u) : "memory");
	}
	if (threadIdx.x == 0)
	{
		asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_addr) : "memory");
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)), "r"((uint32_t)UP_N) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem = tmem_slot;

	if (threadIdx.x == 0)
	{
		auto desc = [](uint32_t addr)
		{
			return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32)
					| ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
		};
		const uint32_t idesc = (2u << 4) | ((uint32_t)(UP_N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
		uint32_t phase = 0;
		bool ok = true;
		for (int it = 0; it < iters && ok; ++it)
		{
			#pragma unroll
			for (int k = 0; k < 4; ++k)
			{
				const uint64_t a = desc(base + k * 32);
				const uint64_t b = desc(base + 128 * 128 + k * 32);
				asm volatile(
					"{\n\t.reg .pred p;\n\t"
					"setp.ne.b32 p, %4, 0;\n\t"
					"tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
					:: "r"(tmem), "l"(a), "l"(b), "r"(idesc), "r"((it | k) ? 1u : 0u), "r"(0u) : "memory");
			}
			if ((it & 15) == 15 || it == iters - 1)
			{
				asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar_addr) : "memory");
				ok = false;
				for (uint32_t spin = 0; spin < UP_SPIN_LIMIT; ++spin)
				{
					uint32_t done;
					asm volatile(
						"{\n\t.reg .pred p;\n\t"
						"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
						"selp.u32 %0, 1, 0, p;\n\t}"
						: "=r"(done) : "r"(bar_addr), "r"(phase) : "memory");
					if (done) { ok = true; break; }
				}
				phase ^= 1u;
			}
		}
		if (!ok) { atomicAdd(timeouts, 1); }
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 0)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)UP_N) : "memory");
	}
}


// The same for the kernel's own instruction: tcgen05.mma kind::mxf4 (e2m1 operands, ue8m0 scale factors of 2^0 in tensor
// memory), M=128, N=256, K=64, counted as 2*M*N*K per instruction.
constexpr int UPF_TMEM_COLS = 512;
constexpr int UPF_SF_COL = 256;

__global__ void __launch_bounds__(UP_THREADS)
umma_mxf4_peak_kernel(int iters, int * timeouts)
{
	extern __shared__ uint8_t up_smem_raw[];
	__shared__ uint64_t bar;
	__shared__ uint32_t tmem_slot;
	const uint32_t base = ((uint32_t)__cvta_generic_to_shared(up_smem_raw) + 1023u) & ~1023u;
	const uint32_t bar_addr = (uint32_t)__cvta_generic_to_shared(&bar);
	const int warp = threadIdx.x >> 5;

	for (int i = threadIdx.x; i < (128 + UP_N) * 128 / 16; i += UP_THREADS)
	{
		asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" :: "r"(base + i * 16), "r"(0x2A2A2A2Au) : "memory");
	}
	if (threadIdx.x == 0)
	{
		asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_addr) : "memory");
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)), "r"((uint32_t)UPF_TMEM_COLS) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem = tmem_slot;
	{
		// scale factors: 16 columns of 2^0 on this warp's 32 lanes
		const uint32_t taddr = tmem + (uint32_t)UPF_SF_COL + ((uint32_t)(warp * 32) << 16);
		asm volatile(
			"tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
			:: "r"(taddr), "r"(0x7F7F7F7Fu) : "memory");
		asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

	if (threadIdx.x == 0)
	{
		auto desc = [](uint32_t addr)
		{
			return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32)
					| ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
		};
		const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(UP_N >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24);
		const uint32_t sfa = tmem + (uint32_t)UPF_SF_COL, sfb = sfa + 8;
		uint32_t phase = 0;
		bool ok = true;
		for (int it = 0; it < iters && ok; ++it)
		{
			#pragma unroll
			for (int k = 0; k < 4; ++k)
			{
				const uint64_t a = desc(base + k * 32);
				const uint64_t b = desc(base + 128 * 128 + k * 32);
				asm volatile(
					"{\n\t.reg .pred p;\n\t"
					"setp.ne.b32 p, %4, 0;\n\t"
					"tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
					:: "r"(tmem), "l"(a), "l"(b), "r"(idesc), "r"((it | k) ? 1u : 0u), "r"(sfa), "r"(sfb) : "memory");
			}
			if ((it & 15) == 15 || it == iters - 1)
			{
				asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar_addr) : "memory");
				ok = false;
				for (uint32_t spin = 0; spin < UP_SPIN_LIMIT; ++spin)
				{
					uint32_t done;
					asm volatile(
						"{\n\t.reg .pred p;\n\t"
						"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
						"selp.u32 %0, 1, 0, p;\n\t}"
						: "=r"(done) : "r"(bar_addr), "r"(phase) : "memory");
					if (done) { ok = true; break; }
				}
				phase ^= 1u;
			}
		}
		if (!ok) { atomicAdd(timeouts, 1); }
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 0)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t)UPF_TMEM_COLS) : "memory");
	}
}

}  // namespace xnor

using namespace xnor;

static int measure_umma_peak(void (*kernel)(int, int *), double ops_per_mma, int iters, double * gops, double * ms_out)
{
	if (gops == nullptr || ms_out == nullptr) { return XNOR_B200_ERR_NULL; }
	if (iters <= 0 || iters > (1 << 20)) { return XNOR_B200_ERR_INVALID; }
	int rc = ensure_dynamic_smem((const void *)kernel, UP_SMEM);
	if (rc != XNOR_B200_OK) { return rc; }
	int * timeouts = nullptr;
	cudaError_t e = cudaMalloc(&timeouts, sizeof(int));
	if (e != cudaSuccess) { return cuda_fail(e); }
	cudaMemset(timeouts, 0, sizeof(int));
	const int blocks = sm_count();
	cudaEvent_t t0, t1;
	cudaEventCreate(&t0);
	cudaEventCreate(&t1);
	float best = 1e30f;
	for (int rep = 0; rep < 4; ++rep)   // first repetition is the warm-up
	{
		cudaEventRecord(t0, 0);
		kernel<<<blocks, UP_THREADS, UP_SMEM>>>(iters, timeouts);
		cudaEventRecord(t1, 0);
		e = cudaEventSynchronize(t1);
		if (e != cudaSuccess) { break; }
		float ms = 0.0f;
		cudaEventElapsedTime(&ms, t0, t1);
		if (rep > 0 && ms < best) { best = ms; }
	}
	int h_timeouts = 0;
	if (e == cudaSuccess) { e = cudaMemcpy(&h_timeouts, timeouts, sizeof(int), cudaMemcpyDeviceToHost); }
	cudaEventDestroy(t0);
	cudaEventDestroy(t1);
	cudaFree(timeouts);
	if (e != cudaSuccess) { return cuda_fail(e); }
	if (h_timeouts != 0) { return XNOR_B200_ERR_INVALID; }
	const double ops = (double)blocks * (double)iters * 4.0 * ops_per_mma;
	*ms_out = best;
	*gops = ops / (best * 1e-3) / 1e9;
	return XNOR_B200_OK;
}

extern "C" int xnor_b200_measure_umma_i8_peak(int iters, double * gops, double * ms_out)
{
	return measure_umma_peak(umma_i8_peak_kernel, 2.0 * 128 * UP_N * 32, iters, gops, ms_out);
}

extern "C" int xnor_b200_measure_umma_mxf4_peak(int iters, double * gops, double * ms_out)
{
	return measure_umma_peak(umma_mxf4_peak_kernel, 2.0 * 128 * UP_N * 64, iters, gops, ms_out);
}
