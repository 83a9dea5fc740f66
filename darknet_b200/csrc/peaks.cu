// On-device measurement of the two candidate rooflines of the XNOR GEMM: the integer pipe
// (XOR + POPC + ADD on 32-bit words) and the legacy 1-bit tensor path (mma.sync b1 xor.popc).
// Neither figure is published for this GPU, so the benchmark measures them where it runs.
// Both loops work on registers only; every thread writes one word at the end so the compiler keeps them.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int PEAK_THREADS = 256;

// Same instruction mix as the GEMM inner loop: an 8x8 register tile, 64 (xor, popc, add) per step,
// operands refreshed with a handful of adds so nothing is loop-invariant.
__global__ void __launch_bounds__(PEAK_THREADS)
popc_peak_kernel(int iters, uint32_t * sink)
{
	uint32_t a[8], b[8];
	int acc[8][8];
	#pragma unroll
	for (int i = 0; i < 8; ++i)
	{
		a[i] = threadIdx.x * 2654435761u + i * 40503u + blockIdx.x;
		b[i] = threadIdx.x * 2246822519u + i * 3266489917u + blockIdx.x * 7u;
		#pragma unroll
		for (int j = 0; j < 8; ++j) { acc[i][j] = 0; }
	}
	for (int it = 0; it < iters; ++it)
	{
		#pragma unroll
		for (int i = 0; i < 8; ++i)
		{
			#pragma unroll
			for (int j = 0; j < 8; ++j) { acc[i][j] += __popc(a[i] ^ b[j]); }
		}
		#pragma unroll
		for (int i = 0; i < 8; ++i) { a[i] += 0x9e3779b9u; b[i] += 0x7f4a7c15u; }
	}
	uint32_t s = 0;
	#pragma unroll
	for (int i = 0; i < 8; ++i)
	{
		#pragma unroll
		for (int j = 0; j < 8; ++j) { s += (uint32_t)acc[i][j]; }
	}
	sink[blockIdx.x * PEAK_THREADS + threadIdx.x] = s;
}

// One warp issues 8 independent m16n8k256 b1 xor.popc MMAs per step (8 accumulator fragments).
__global__ void __launch_bounds__(PEAK_THREADS)
bmma_peak_kernel(int iters, uint32_t * sink)
{
	uint32_t a0 = threadIdx.x * 2654435761u, a1 = a0 ^ 0x55555555u, a2 = a0 * 3u, a3 = a0 + 17u;
	uint32_t b0 = threadIdx.x * 2246822519u + blockIdx.x, b1 = b0 ^ 0x33333333u;
	int c[8][4];
	#pragma unroll
	for (int u = 0; u < 8; ++u) { c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0; }
	for (int it = 0; it < iters; ++it)
	{
		#pragma unroll
		for (int u = 0; u < 8; ++u)
		{
			asm volatile(
				"mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.xor.popc "
				"{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
				: "+r"(c[u][0]), "+r"(c[u][1]), "+r"(c[u][2]), "+r"(c[u][3])
				: "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0 + u), "r"(b1));
		}
		a0 += 0x9e3779b9u;
	}
	uint32_t s = 0;
	#pragma unroll
	for (int u = 0; u < 8; ++u) { s += (uint32_t)(c[u][0] + c[u][1] + c[u][2] + c[u][3]); }
	sink[blockIdx.x * PEAK_THREADS + threadIdx.x] = s;
}

static int run_peak(bool bmma, int iters, double * gops, double * ms_out)
{
	if (gops == nullptr || ms_out == nullptr) { return XNOR_B200_ERR_NULL; }
	if (iters <= 0 || iters > (1 << 24)) { return XNOR_B200_ERR_INVALID; }
	const int blocks = sm_count() * 4;
	uint32_t * sink = nullptr;
	cudaError_t e = cudaMalloc(&sink, (size_t)blocks * PEAK_THREADS * sizeof(uint32_t));
	if (e != cudaSuccess) { return cuda_fail(e); }
	cudaEvent_t t0, t1;
	cudaEventCreate(&t0);
	cudaEventCreate(&t1);
	float best = 1e30f;
	for (int rep = 0; rep < 4; ++rep)   // first repetition is the warm-up
	{
		cudaEventRecord(t0, 0);
		if (bmma) { bmma_peak_kernel<<<blocks, PEAK_THREADS>>>(iters, sink); }
		else      { popc_peak_kernel<<<blocks, PEAK_THREADS>>>(iters, sink); }
		cudaEventRecord(t1, 0);
		e = cudaEventSynchronize(t1);
		if (e != cudaSuccess) { break; }
		float ms = 0.0f;
		cudaEventElapsedTime(&ms, t0, t1);
		if (rep > 0 && ms < best) { best = ms; }
	}
	cudaEventDestroy(t0);
	cudaEventDestroy(t1);
	cudaFree(sink);
	if (e != cudaSuccess) { return cuda_fail(e); }
	const double threads = (double)blocks * PEAK_THREADS;
	const double binops = bmma
		? threads / 32.0 * (double)iters * 8.0 * (2.0 * 16 * 8 * 256)
		: threads * (double)iters * 64.0 * 64.0;
	*ms_out = best;
	*gops = binops / (best * 1e-3) / 1e9;
	return XNOR_B200_OK;
}

}  // namespace xnor

extern "C" int xnor_b200_measure_popc_peak(int iters, double * gops, double * ms) { return xnor::run_peak(false, iters, gops, ms); }
extern "C" int xnor_b200_measure_bmma_peak(int iters, double * gops, double * ms) { return xnor::run_peak(true, iters, gops, ms); }
