// Float 1x1 / stride-1 convolutions at batch (the heads behind the xnor path: yolo and region heads, 255..1024 filters
// over 256..1024 channels and tens of thousands of pixels) on the tcgen05 tensor cores, at fp32 accuracy.
//
// Replaces, for those layers, the float branch of forward_convolutional_layer_gpu (src-lib/convolutional_kernels.cu:373-434:
// a cuBLAS/cuDNN GEMM per image) + add_bias_gpu + activate_array_ongpu.  out[b][f][p] = bias[f] + sum_c w[f][c] * x[b][c][p].
//
// The tensor core multiplies tf32 (10 mantissa bits).  Every fp32 operand value v is therefore split into hi = v with the low
// 13 mantissa bits cleared (exactly a tf32) and lo = v - hi (exact in fp32, magnitude <= 2^-10 |v|), and three products are
// accumulated per pair: hi*hi + lo*hi + hi*lo.  What is dropped (lo*lo and the bits of lo below tf32) is below 2^-20 of each
// product.  The tensor core adds into its fp32 accumulator without rounding to nearest (measured: the error of a sum grows
// linearly with the number of accumulating instructions, ~1e-7 of the sum per instruction), so consecutive K blocks go to four
// accumulators in turn (all 512 tensor-memory columns) and the epilogue adds the four partial sums with ordinary fp32
// additions: 1024 channels come out within 2e-5 of an fp64 convolution for results of magnitude 1 -- far inside what the
// reference's own GPU path does (it asks cuDNN for tensor-op math, i.e. single tf32 products, on every convolution:
// src-lib/convolutional_layer.cpp:350).
//
// Same skeleton as xnor_gemm_tc.cu: one CTA = 128 pixels (TMEM lanes; the batch is folded into the pixel index) x 128
// filters (TMEM columns), warp 0 allocates tensor memory and one lane issues, 16 producer warps -- two threads per operand
// row, 16 channels of every K block each (pixel row: one coalesced load per channel across the warp; filter row: 64
// contiguous bytes) -- split their values and write hi and lo straight into K-major SWIZZLE_128B tiles (32 tf32 = one 128-byte row); 12
// tcgen05.mma.kind::tf32 (M=128, N=128, K=8) per K block of 32 channels; the same warps then add the bias, apply leaky and
// store 32 consecutive pixels of one filter per warp-store.  Every barrier wait is bounded (status word shared with the
// xnor tensor-core kernels).
#include "tc_common.cuh"

namespace xnor
{

constexpr int FT_NF = 128;                                 // filters per tile
constexpr int FT_ACCS = 4;                                 // accumulators that take the K blocks in turn
constexpr int FT_STAGES = 3;
constexpr int FT_TILE_BYTES = 128 * 128;                   // 128 rows x 32 tf32
constexpr int FT_STAGE_BYTES = 4 * FT_TILE_BYTES;          // pixel hi, pixel lo, filter hi, filter lo
constexpr int FT_SMEM_BYTES = FT_STAGES * FT_STAGE_BYTES + 1024;
constexpr int FT_TPR = 2;                                  // producer threads per operand row: each takes 32 / FT_TPR channels of a K block
constexpr int FT_CH = 32 / FT_TPR;
constexpr int FT_PRODUCER_WARPS = 8 * FT_TPR;
constexpr int FT_THREADS = 32 + 32 * FT_PRODUCER_WARPS;

struct FtParams
{
	const float * x;      // [batch][C][HW]
	const float * w;      // [N][C]
	const float * bias;   // [N] or nullptr
	float * out;          // [batch][N][HW]
	int C, HW, N;
	int total;            // batch * HW
	int kblocks;          // ceil(C / 32)
	int leaky;
	int tiles_f;
	int w_vec;            // 1: weight rows may be read with 16-byte loads
	int * status;
	uint32_t spin_limit;
};

// A thread's part of one operand row of one K block: FT_CH fp32 values -> their 16-byte chunks in the row of the hi tile and
// of the lo tile (chunk c of row r at chunk position c ^ (r % 8); row_swz has the row's swizzle term and the part's first
// chunk folded in).
__device__ __forceinline__ void split_row(uint32_t row_swz_hi, uint32_t lo_offset, const float (&v)[FT_CH])
{
	#pragma unroll
	for (int c = 0; c < FT_CH / 4; ++c)
	{
		uint32_t hi[4], lo[4];
		#pragma unroll
		for (int j = 0; j < 4; ++j)
		{
			const uint32_t bits = __float_as_uint(v[4 * c + j]);
			hi[j] = bits & 0xFFFFE000u;
			lo[j] = __float_as_uint(__fsub_rn(v[4 * c + j], __uint_as_float(hi[j])));
		}
		const uint32_t addr = row_swz_hi ^ (uint32_t)(c << 4);
		asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
		asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr + lo_offset), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
	}
}

__global__ void __launch_bounds__(FT_THREADS, 1)
float_conv_tc_kernel(const FtParams p)
{
	extern __shared__ uint8_t ft_smem_raw[];
	__shared__ uint64_t bar_full[FT_STAGES];
	__shared__ uint64_t bar_empty[FT_STAGES];
	__shared__ uint64_t bar_done;
	__shared__ uint32_t tmem_base_slot;
	__shared__ float s_bias[FT_NF];
	__shared__ int s_failed_storage;
	volatile int * s_failed = &s_failed_storage;

	const int tid = threadIdx.x;
	const int warp = tid >> 5;
	const int lane = tid & 31;
	const uint32_t ring = (smem_u32(ft_smem_raw) + 1023u) & ~1023u;
	const int tile_p = blockIdx.x / p.tiles_f;
	const int f0 = (blockIdx.x - tile_p * p.tiles_f) * FT_NF;
	const int g0 = tile_p * TC_PIX;                          // first pixel of the tile, batch folded in

	if (tid == 0)
	{
		for (int s = 0; s < FT_STAGES; ++s)
		{
			mbar_init(&bar_full[s], FT_PRODUCER_WARPS);
			mbar_init(&bar_empty[s], 1);
		}
		mbar_init(&bar_done, 1);
		s_failed_storage = 0;
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0)
	{
		asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
				:: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)(FT_ACCS * FT_NF)) : "memory");
		asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
	}
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const uint32_t tmem_base = tmem_base_slot;

	if (warp == 0)
	{
		if (lane == 0)
		{
			// instruction descriptor: D = f32, A = B = tf32, both K-major, N = 128, M = 128
			const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(FT_NF >> 3) << 17) | ((uint32_t)(TC_PIX >> 4) << 24);
			bool ok = true;
			for (int kb = 0; kb < p.kblocks && ok; ++kb)
			{
				const int s = kb % FT_STAGES;
				ok = mbar_wait(&bar_full[s], (uint32_t)((kb / FT_STAGES) & 1), s_failed, p.spin_limit);
				if (!ok) { break; }
				asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
				const uint32_t a_hi = ring + (uint32_t)s * FT_STAGE_BYTES;
				const uint32_t a_lo = a_hi + FT_TILE_BYTES;
				const uint32_t b_hi = a_hi + 2 * FT_TILE_BYTES;
				const uint32_t b_lo = a_hi + 3 * FT_TILE_BYTES;
				#pragma unroll
				for (int k = 0; k < 4; ++k)                       // 8 tf32 = 32 bytes of every row per instruction
				{
					#pragma unroll
					for (int term = 0; term < 3; ++term)          // the two small terms first, the large one last
					{
						const uint64_t adesc = make_smem_desc((term == 0 ? a_lo : a_hi) + k * 32);
						const uint64_t bdesc = make_smem_desc((term == 1 ? b_lo : b_hi) + k * 32);
						const uint32_t accumulate = (kb >= FT_ACCS || k > 0 || term > 0) ? 1u : 0u;
						asm volatile(
							"{\n\t.reg .pred p;\n\t"
							"setp.ne.b32 p, %4, 0;\n\t"
							"tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
							:: "r"(tmem_base + (uint32_t)((kb % FT_ACCS) * FT_NF)), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
					}
				}
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
		// ---- producers: per part (FT_CH channels of every K block) four warps of pixel rows and four of filter rows -------
		const int part = (warp - 1) >> 3;
		const int r = (tid - 32) - part * 256;
		const bool is_pix = r < TC_PIX;
		const int row = is_pix ? r : r - TC_PIX;
		const uint32_t row_swz0 = (ring + (is_pix ? 0u : 2u * FT_TILE_BYTES) + (uint32_t)row * 128u)
				^ ((uint32_t)((row & 7) ^ (part * (FT_CH / 4))) << 4);
		const int g = g0 + row;
		const int f = f0 + row;
		const bool row_ok = is_pix ? (g < p.total) : (f < p.N);
		const int img = (is_pix && row_ok) ? g / p.HW : 0;
		const int pix = (is_pix && row_ok) ? g - img * p.HW : 0;
		// element c of the row is base[c * stride]
		const float * base = is_pix ? p.x + (size_t)img * p.C * p.HW + pix : p.w + (size_t)(row_ok ? f : 0) * p.C;
		const size_t stride = is_pix ? (size_t)p.HW : 1;
		float nxt[FT_CH];
		auto fetch = [&](int kb)
		{
			const int c0 = kb * 32 + part * FT_CH;
			if (!is_pix && p.w_vec && row_ok && c0 + FT_CH <= p.C)
			{
				#pragma unroll
				for (int q = 0; q < FT_CH / 4; ++q)
				{
					const float4 t = __ldg(reinterpret_cast<const float4 *>(base + c0) + q);
					nxt[4 * q] = t.x; nxt[4 * q + 1] = t.y; nxt[4 * q + 2] = t.z; nxt[4 * q + 3] = t.w;
				}
				return;
			}
			#pragma unroll
			for (int k = 0; k < FT_CH; ++k)
			{
				nxt[k] = (row_ok && c0 + k < p.C) ? __ldg(base + (size_t)(c0 + k) * stride) : 0.0f;
			}
		};
		fetch(0);
		bool ok = true;
		for (int kb = 0; kb < p.kblocks; ++kb)
		{
			const int s = kb % FT_STAGES;
			float cur[FT_CH];
			#pragma unroll
			for (int k = 0; k < FT_CH; ++k) { cur[k] = nxt[k]; }
			if (kb + 1 < p.kblocks) { fetch(kb + 1); }
			if (kb >= FT_STAGES)
			{
				ok = mbar_wait(&bar_empty[s], (uint32_t)((kb / FT_STAGES - 1) & 1), s_failed, p.spin_limit);
				if (!ok) { break; }
			}
			split_row(row_swz0 + (uint32_t)s * FT_STAGE_BYTES, (uint32_t)FT_TILE_BYTES, cur);
			asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
			__syncwarp();
			if (lane == 0) { mbar_arrive(&bar_full[s]); }
		}
		if (!is_pix && part == 0) { s_bias[row] = (row_ok && p.bias != nullptr) ? __ldg(p.bias + f) : 0.0f; }
	}

	if (tid == 0) { mbar_wait<64>(&bar_done, 0, s_failed, p.spin_limit); }
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
	const bool failed = (*s_failed != 0);

	if (!failed && warp != 0)
	{
		// warp w reads the TMEM lanes of quarter w % 4; the warps of a quarter share the four 32-filter chunks
		const int quarter = warp & 3;
		const int share = (warp - 1) >> 2;
		constexpr int SHARES = FT_PRODUCER_WARPS / 4;
		const int g = g0 + quarter * 32 + lane;
		const bool col_ok = g < p.total;
		const int img = col_ok ? g / p.HW : 0;
		const int pix = col_ok ? g - img * p.HW : 0;
		float * out_pix = p.out + ((size_t)img * p.N + f0) * p.HW + pix;
		const float slope = p.leaky ? 0.1f : 1.0f;
		#pragma unroll 1
		for (int chunk = share; chunk < FT_NF / 32; chunk += SHARES)
		{
			// the partial sums of the accumulators that were used, added in fp32
			float acc[32];
			const int used = min(FT_ACCS, p.kblocks);
			#pragma unroll 1
			for (int a = 0; a < used; ++a)
			{
				uint32_t d[32];
				tmem_load<32>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * FT_NF + chunk * 32), d);
				asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
				#pragma unroll
				for (int j = 0; j < 32; ++j) { acc[j] = (a == 0) ? __uint_as_float(d[j]) : __fadd_rn(acc[j], __uint_as_float(d[j])); }
			}
			if (!col_ok) { continue; }
			#pragma unroll
			for (int j = 0; j < 32; ++j)
			{
				const int fl = chunk * 32 + j;
				if (f0 + fl < p.N)
				{
					float v = __fadd_rn(acc[j], s_bias[fl]);
					v = fmaxf(v, __fmul_rn(v, slope));
					out_pix[(size_t)fl * p.HW] = v;
				}
			}
		}
	}
	else if (failed && tid == 0)
	{
		atomicExch(p.status, 1);
	}

	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
	__syncthreads();
	if (warp == 0)
	{
		asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)(FT_ACCS * FT_NF)) : "memory");
	}
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_float_conv_1x1_tc(const xnor_b200_conv_desc * desc, const float * input, const float * weights,
		const float * biases, float * output, void * stream)
{
	if (desc == nullptr || input == nullptr || weights == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (desc->size != 1 || desc->stride != 1 || desc->pad != 0) { return XNOR_B200_ERR_INVALID; }
	const long long total = (long long)desc->batch * desc->h * desc->w;
	if (total > 0x7fffffffLL - TC_PIX) { return XNOR_B200_ERR_TOO_LARGE; }
	FtParams p;
	p.x = input; p.w = weights; p.bias = biases; p.out = output;
	p.C = desc->c; p.HW = desc->h * desc->w; p.N = desc->n;
	p.total = (int)total;
	p.kblocks = (desc->c + 31) / 32;
	p.leaky = (desc->activation == XNOR_B200_LEAKY) ? 1 : 0;
	p.tiles_f = (desc->n + FT_NF - 1) / FT_NF;
	p.w_vec = (desc->c % 4 == 0 && (((uintptr_t)weights) & 15u) == 0) ? 1 : 0;
	TcParams tp = TcParams();
	rc = tc_fill_launch_fields(tp);
	if (rc != XNOR_B200_OK) { return rc; }
	p.status = tp.status;
	p.spin_limit = tp.spin_limit;
	const long long grid = (long long)p.tiles_f * ((total + TC_PIX - 1) / TC_PIX);
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	rc = ensure_dynamic_smem((const void *)float_conv_tc_kernel, FT_SMEM_BYTES);
	if (rc != XNOR_B200_OK) { return rc; }
	float_conv_tc_kernel<<<(unsigned)grid, FT_THREADS, FT_SMEM_BYTES, (cudaStream_t)stream>>>(p);
	return check_launch();
}
