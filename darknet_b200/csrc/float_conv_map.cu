// fp32 convolution for the float layers BEHIND the xnor path: many channels on a small feature map (the 3x3
// 256->512 convolution on 13x13 and the 1x1 convolutions in front of the yolo heads), bias and leaky/linear fused.
//
// Stands in for the float branch of forward_convolutional_layer_gpu (src-lib/convolutional_kernels.cu:373-434:
// cuDNN, or im2col + cuBLAS sgemm), add_bias_gpu (src-lib/blas_kernels.cu) and activate_array_ongpu
// (src-lib/activation_kernels.cu:34).  At batch 1 such a layer is a 512 x 169 x 2304 product: far too few output
// values to fill the GPU with one value per thread, and library kernels run it as a handful of large CTAs (about
// 70 us for a product that is 5 us of FFMA work).  This kernel spreads it over the whole chip instead:
//   grid = (pixel tiles x images, filter tiles of 32, K splits), the K splits of one tile form a thread-block
//   cluster; every CTA runs a 3-stage cp.async pipeline over its channels (weights pre-blocked at load time so a
//   stage is one contiguous copy; the input staged as a zero-bordered image so a tap is a constant offset), each
//   thread holds 8 filters x 6 pixels in registers, and the partial sums of a cluster are added in rank order
//   through distributed shared memory (deterministic; no atomics), then bias, activation and one coalesced store.
// fp32 FMA throughout; the summation order is (split, channel, ky, kx), so results agree with cuDNN/cuBLAS to
// rounding, not bit for bit.
#include "xnor_common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace xnor
{

// 16 warps per CTA: K groups (each takes every KG-th channel of a stage) x 2 filter halves x (1 or 2) pixel halves.
// A warp covers 16 filters x 96 pixels, a lane 8 filters x 6 pixels: per K value it reads two 16-byte weight
// vectors (two addresses per warp) and six inputs (16 neighbouring addresses per warp, no bank conflict), 8
// shared-memory wavefronts for 48 FFMA, which keeps the FMA pipe, not the load/store unit, the limiter.  The staged
// image has a compile-time row pitch (16 or 32 floats), so every tap is an immediate offset of one load.
constexpr int FM_THREADS = 512;
constexpr int FM_FT = 32;                  // filters per CTA
constexpr int FM_PJ = 6;                   // pixels per thread: slots half*96 + (lane & 15) + 16 j
constexpr int FM_STAGES = 3;
constexpr int FM_MAX_DEVICES = 64;

struct FloatMapParams
{
	const float * in;        // [batch][C][H*W]
	const float * wblk;      // [filter tile][K][32]
	const float * bias;      // [N] or nullptr
	float * out;             // [batch][N][H*W]
	int C, H, W, N;
	int K;                   // C * taps
	int ptiles;              // pixel tiles per image
	int splits;              // cluster size along z
	int chans_per_split;
	int leaky;
	int yolo_entries;        // > 0: the layer feeds a [yolo] head with this many entries per anchor (4 + 1 + classes): logistic on
	                         //      every entry but w, h (entries 2, 3), as forward_yolo_layer_gpu does right after this layer
};

__device__ __forceinline__ void cp_async_4z(float * smem_dst, const float * gmem_src, bool valid)
{
	const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
	const int n = valid ? 4 : 0;
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" :: "r"(d), "l"(gmem_src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_16f(float * smem_dst, const float * gmem_src)
{
	const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

// KS = 3: stride 1, pad 1, staged as a zero-bordered image of PITCH floats per row (PITCH 16: maps up to 14x14,
// 16 rows; PITCH 32: up to 30x30, 32 rows).  KS = 1: stride 1, pad 0, PITCH unused (the PT pixel slots are staged).
// PT = pixel slots per CTA (96 or 192).
template <int KS, int PITCH, int PT, int CKP>
struct FloatMapShape
{
	static constexpr int TAPS = KS * KS;
	static constexpr int CK = CKP;                                      // channels per pipeline stage
	static constexpr int CKT = CK * TAPS;                               // K values per stage
	static constexpr int AREA = (KS == 3) ? PITCH * PITCH : PT;         // staged floats per channel
	static constexpr int PH = PT / 96;                                  // pixel halves
	static constexpr int KG = 16 / (2 * PH);                            // K groups: 4 or 8
	static constexpr int STAGE_FLOATS = CKT * FM_FT + CK * AREA;
	static constexpr size_t SMEM = (size_t)((STAGE_FLOATS * FM_STAGES > FM_FT * PT) ? STAGE_FLOATS * FM_STAGES : FM_FT * PT) * sizeof(float);
	static constexpr int MAXE = (AREA + FM_THREADS - 1) / FM_THREADS;   // staged elements per channel per thread
};

template <int KS, int PITCH, int PT, int CKP>
__global__ void __launch_bounds__(FM_THREADS)
float_conv_map_kernel(const FloatMapParams p)
{
	using SH = FloatMapShape<KS, PITCH, PT, CKP>;
	constexpr int TAPS = SH::TAPS, CK = SH::CK, CKT = SH::CKT, AREA = SH::AREA, KG = SH::KG, MAXE = SH::MAXE;
	constexpr int STAGE_FLOATS = SH::STAGE_FLOATS;
	extern __shared__ __align__(16) float s_mem[];

	const int tid = threadIdx.x;
	const int lane = tid & 31;
	const int warp = tid >> 5;
	const int f_first = (warp & 1) * 16 + (lane >> 4) * 8;             // first of this thread's 8 filters inside the tile
	const int slot0 = ((warp >> 1) % SH::PH) * 96 + (lane & 15);       // first of its 6 pixel slots (stride 16)
	const int kg = warp / (2 * SH::PH);                                // K group
	const int img = blockIdx.x / p.ptiles;
	const int pt = blockIdx.x - img * p.ptiles;
	const int mt = blockIdx.y;
	const int split = blockIdx.z;
	const int HW = p.H * p.W;

	// which global element (offset inside one channel plane) each staged element of this thread comes from
	int eoff[MAXE];
	#pragma unroll
	for (int i = 0; i < MAXE; ++i)
	{
		const int e = tid + i * FM_THREADS;
		int off = -1;
		if (KS == 3)
		{
			const int py = e / PITCH;
			const int px = e % PITCH;
			if (e < AREA && py >= 1 && py <= p.H && px >= 1 && px <= p.W) { off = (py - 1) * p.W + (px - 1); }
		}
		else
		{
			const int q = pt * PT + e;
			if (e < AREA && q < HW) { off = q; }
		}
		eoff[i] = off;
	}
	// where each of this thread's pixels starts inside a staged channel
	int base[FM_PJ];
	#pragma unroll
	for (int j = 0; j < FM_PJ; ++j)
	{
		const int slot = slot0 + 16 * j;
		if (KS == 3)
		{
			const int q = pt * PT + slot;
			const int y = (q < HW) ? q / p.W : 0;
			const int x = (q < HW) ? q - y * p.W : 0;
			base[j] = y * PITCH + x;
		}
		else { base[j] = slot; }
	}

	const float * in_img = p.in + (size_t)img * p.C * HW;
	const int c_begin = split * p.chans_per_split;
	const int nq = p.chans_per_split / CK;

	auto load_stage = [&](int q, int s)
	{
		float * sw = s_mem + (size_t)s * STAGE_FLOATS;
		float * sx = sw + CKT * FM_FT;
		const int c0 = c_begin + q * CK;
		const float * wsrc = p.wblk + ((size_t)mt * p.K + (size_t)c0 * TAPS) * FM_FT;
		for (int v = tid; v < CKT * FM_FT / 4; v += FM_THREADS) { cp_async_16f(sw + v * 4, wsrc + v * 4); }
		#pragma unroll 4
		for (int c = 0; c < CK; ++c)
		{
			const float * plane = in_img + (size_t)(c0 + c) * HW;
			#pragma unroll
			for (int i = 0; i < MAXE; ++i)
			{
				const int e = tid + i * FM_THREADS;
				if (e < AREA) { cp_async_4z(sx + c * AREA + e, (eoff[i] >= 0) ? plane + eoff[i] : in_img, eoff[i] >= 0); }
			}
		}
	};

	// accumulators as filter pairs: one packed FMA (fma.rn.f32x2, two independent IEEE FMAs) per pair and pixel
	float2 acc2[4][FM_PJ];
	#pragma unroll
	for (int f = 0; f < 4; ++f)
	{
		#pragma unroll
		for (int j = 0; j < FM_PJ; ++j) { acc2[f][j] = make_float2(0.0f, 0.0f); }
	}

	#pragma unroll
	for (int s = 0; s < FM_STAGES - 1; ++s)
	{
		if (s < nq) { load_stage(s, s); }
		cp_commit();
	}
	for (int q = 0; q < nq; ++q)
	{
		cp_wait<FM_STAGES - 2>();
		__syncthreads();
		if (q + FM_STAGES - 1 < nq) { load_stage(q + FM_STAGES - 1, (q + FM_STAGES - 1) % FM_STAGES); }
		cp_commit();
		const float * sw = s_mem + (size_t)(q % FM_STAGES) * STAGE_FLOATS + f_first + kg * TAPS * FM_FT;
		const float * sx = s_mem + (size_t)(q % FM_STAGES) * STAGE_FLOATS + CKT * FM_FT + kg * AREA;
		const float * sxj[FM_PJ];
		#pragma unroll
		for (int j = 0; j < FM_PJ; ++j) { sxj[j] = sx + base[j]; }
		#pragma unroll
		for (int cc = 0; cc < CK / KG; ++cc)                 // this K group's channels: kg, kg + KG, ...
		{
			#pragma unroll
			for (int t = 0; t < TAPS; ++t)
			{
				const float4 w0 = *reinterpret_cast<const float4 *>(sw + (cc * KG * TAPS + t) * FM_FT);
				const float4 w1 = *reinterpret_cast<const float4 *>(sw + (cc * KG * TAPS + t) * FM_FT + 4);
				#pragma unroll
				for (int j = 0; j < FM_PJ; ++j)
				{
					const float xv = sxj[j][cc * KG * AREA + ((KS == 3) ? (t / KS) * PITCH + (t % KS) : 0)];
					const float2 xx = make_float2(xv, xv);
					acc2[0][j] = __ffma2_rn(make_float2(w0.x, w0.y), xx, acc2[0][j]);
					acc2[1][j] = __ffma2_rn(make_float2(w0.z, w0.w), xx, acc2[1][j]);
					acc2[2][j] = __ffma2_rn(make_float2(w1.x, w1.y), xx, acc2[2][j]);
					acc2[3][j] = __ffma2_rn(make_float2(w1.z, w1.w), xx, acc2[3][j]);
				}
			}
		}
	}
	cp_wait<0>();
	__syncthreads();

	// partial sums of this split: [32 filters][PT slots] at the start of shared memory; the K groups add theirs one
	// after the other (same thread-to-element mapping in every group, so only the barrier orders them)
	float * s_part = s_mem;
	#pragma unroll
	for (int g = 0; g < KG; ++g)
	{
		if (kg == g)
		{
			#pragma unroll
			for (int f = 0; f < 8; ++f)
			{
				#pragma unroll
				for (int j = 0; j < FM_PJ; ++j)
				{
					float * dst = s_part + (f_first + f) * PT + slot0 + 16 * j;
					const float a = (f & 1) ? acc2[f >> 1][j].y : acc2[f >> 1][j].x;
					*dst = (g == 0) ? a : *dst + a;
				}
			}
		}
		if (g + 1 < KG) { __syncthreads(); }
	}
	const int S = p.splits;
	const float * parts[8];
	if (S > 1)
	{
		cg::cluster_group cluster = cg::this_cluster();
		cluster.sync();
		#pragma unroll
		for (int r = 0; r < 8; ++r) { parts[r] = (r < S) ? cluster.map_shared_rank(s_part, r) : s_part; }
	}
	else
	{
		__syncthreads();
		parts[0] = s_part;
	}
	// rank `split` finishes filters [split*rows, split*rows + rows) of the tile
	const int rows = FM_FT / S;
	for (int o = tid; o < rows * PT; o += FM_THREADS)
	{
		const int fr = o / PT;
		const int slot = o - fr * PT;
		const int ft = split * rows + fr;
		float sum = 0.0f;
		#pragma unroll
		for (int r = 0; r < 8; ++r)
		{
			if (r < S) { sum += parts[r][ft * PT + slot]; }
		}
		const int f = mt * FM_FT + ft;
		const int q = pt * PT + slot;
		if (f < p.N && q < HW)
		{
			if (p.bias != nullptr) { sum += p.bias[f]; }
			if (p.leaky) { sum = (sum > 0.0f) ? sum : sum * 0.1f; }
			if (p.yolo_entries > 0)
			{
				const int e = f % p.yolo_entries;
				if (e != 2 && e != 3) { sum = 1.0f / (1.0f + expf(-sum)); }
			}
			p.out[((size_t)img * p.N + f) * HW + q] = sum;
		}
	}
	if (S > 1) { cg::this_cluster().sync(); }       // nobody leaves while a peer still reads its partial sums
}

// ---- 1x1 layers: one load, one pass -------------------------------------------------------------------------
// A 1x1 convolution on a small map is a tiny matrix product (255 x 169 x 512 for a yolo head): the pipeline, the
// cluster and its two barriers above cost more than the arithmetic.  Here a CTA owns 16 filters x 32 pixels, issues
// ALL of its operand loads at once (K x 16 weights as 16-byte copies out of the blocked layout, K x 32 inputs as 4-byte
// copies: 48 KB for K = 256), waits once, lets each of its 8 warps run over an eighth of the channels (lane = pixel, 16
// accumulators, weights read as broadcasts), and adds the eight partial tiles through shared memory.  One barrier pair,
// no cluster, and enough CTAs (96 for the 13x13 head, 352 for the 26x26 one) to cover the chip in one wave.
constexpr int F1_THREADS = 256;
constexpr int F1_FT = 16;                  // filters per CTA (half of a 32-filter block of the blocked weights)
constexpr int F1_PT = 32;                  // pixels per CTA
constexpr int F1_MAX_K = 512;              // 192 bytes of shared memory per channel: two CTAs per SM at the limit

__global__ void __launch_bounds__(F1_THREADS)
float_conv_1x1_kernel(const FloatMapParams p)
{
	extern __shared__ __align__(16) float s_mem[];
	const int K = p.C;
	float * s_w = s_mem;                    // [K][16]
	float * s_x = s_mem + (size_t)K * F1_FT;  // [K][32]
	const int tid = threadIdx.x;
	const int lane = tid & 31;
	const int warp = tid >> 5;
	const int HW = p.H * p.W;
	const int img = blockIdx.x / p.ptiles;
	const int pt = blockIdx.x - img * p.ptiles;
	const int ft = blockIdx.y;                                    // 16-filter tile
	const int px = pt * F1_PT + lane;
	const float * in_img = p.in + (size_t)img * p.C * HW;
	const float * wsrc = p.wblk + ((size_t)(ft >> 1) * K) * FM_FT + (ft & 1) * F1_FT;   // row k at wsrc + k*32

	for (int v = tid; v < K * (F1_FT / 4); v += F1_THREADS)
	{
		const int k = v >> 2;
		const int q = v & 3;
		cp_async_16f(s_w + k * F1_FT + q * 4, wsrc + (size_t)k * FM_FT + q * 4);
	}
	for (int k = warp; k < K; k += F1_THREADS / 32)
	{
		cp_async_4z(s_x + k * F1_PT + lane, (px < HW) ? in_img + (size_t)k * HW + px : in_img, px < HW);
	}
	cp_commit();
	cp_wait<0>();
	__syncthreads();

	// warp w takes channels w, w + 8, ...
	float2 acc2[F1_FT / 2];                                       // filter pairs: one packed FMA (fma.rn.f32x2) each
	#pragma unroll
	for (int f = 0; f < F1_FT / 2; ++f) { acc2[f] = make_float2(0.0f, 0.0f); }
	#pragma unroll 4
	for (int k = warp; k < K; k += F1_THREADS / 32)
	{
		const float xv = s_x[k * F1_PT + lane];
		const float2 xx = make_float2(xv, xv);
		const float4 * wr = reinterpret_cast<const float4 *>(s_w + k * F1_FT);
		#pragma unroll
		for (int q = 0; q < 4; ++q)
		{
			const float4 w = wr[q];
			acc2[2 * q] = __ffma2_rn(make_float2(w.x, w.y), xx, acc2[2 * q]);
			acc2[2 * q + 1] = __ffma2_rn(make_float2(w.z, w.w), xx, acc2[2 * q + 1]);
		}
	}
	float acc[F1_FT];
	#pragma unroll
	for (int f = 0; f < F1_FT / 2; ++f) { acc[2 * f] = acc2[f].x; acc[2 * f + 1] = acc2[f].y; }
	__syncthreads();                                              // operands are dead: reuse the front of shared memory
	float * s_part = s_mem;                                       // [8 warps][16 filters][32 pixels]
	#pragma unroll
	for (int f = 0; f < F1_FT; ++f) { s_part[(warp * F1_FT + f) * F1_PT + lane] = acc[f]; }
	__syncthreads();
	for (int o = tid; o < F1_FT * F1_PT; o += F1_THREADS)
	{
		const int fl = o / F1_PT;
		const int sl = o - fl * F1_PT;
		float sum = 0.0f;
		#pragma unroll
		for (int w = 0; w < F1_THREADS / 32; ++w) { sum += s_part[(w * F1_FT + fl) * F1_PT + sl]; }      // fixed order
		const int f = ft * F1_FT + fl;
		const int q = pt * F1_PT + sl;
		if (f < p.N && q < HW)
		{
			if (p.bias != nullptr) { sum += p.bias[f]; }
			if (p.leaky) { sum = (sum > 0.0f) ? sum : sum * 0.1f; }
			if (p.yolo_entries > 0)
			{
				const int e = f % p.yolo_entries;
				if (e != 2 && e != 3) { sum = 1.0f / (1.0f + expf(-sum)); }
			}
			p.out[((size_t)img * p.N + f) * HW + q] = sum;
		}
	}
}

static int launch_float_1x1(const xnor_b200_conv_desc * desc, FloatMapParams p, cudaStream_t stream)
{
	const int HW = desc->h * desc->w;
	p.ptiles = (HW + F1_PT - 1) / F1_PT;
	const int ftiles = (desc->n + F1_FT - 1) / F1_FT;
	const long long gx = (long long)p.ptiles * desc->batch;
	if (gx > 0x7fffffffLL || ftiles > 65535) { return XNOR_B200_ERR_TOO_LARGE; }
	const size_t smem = max((size_t)desc->c * (F1_FT + F1_PT), (size_t)(F1_THREADS / 32) * F1_FT * F1_PT) * sizeof(float);
	int rc = ensure_dynamic_smem((const void *)float_conv_1x1_kernel, smem);
	if (rc != XNOR_B200_OK) { return rc; }
	float_conv_1x1_kernel<<<dim3((unsigned)gx, (unsigned)ftiles, 1), F1_THREADS, smem, stream>>>(p);
	return check_launch();
}

// [n][K] -> [ceil(n/32)][K][32], zero filters behind n
__global__ void float_conv_map_block_weights_kernel(const float * __restrict__ w, float * __restrict__ blk, int N, int K, size_t total)
{
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
	{
		const int fl = (int)(i % FM_FT);
		const size_t rest = i / FM_FT;
		const int k = (int)(rest % K);
		const int mt = (int)(rest / K);
		const int f = mt * FM_FT + fl;
		blk[i] = (f < N) ? w[(size_t)f * K + k] : 0.0f;
	}
}

static int map_conv_shape_ok(const xnor_b200_conv_desc * d)
{
	if (d->stride != 1) { return 0; }
	if (!((d->size == 3 && d->pad == 1) || (d->size == 1 && d->pad == 0))) { return 0; }
	const int ck = (d->size == 3) ? 8 : 32;
	if (d->c % ck != 0) { return 0; }
	if (d->size == 3 && (d->h > 30 || d->w > 30)) { return 0; }
	return 1;
}

// Clusters of `splits` CTAs of this kernel that the device can hold at once (a cluster needs all its SMs in one GPC:
// on a 148-SM part 15 clusters of 8 or 33 of 4 fit, not 18 and 37).  Cached per kernel and cluster size.
template <typename Kern>
static int max_active_clusters(Kern kern, size_t smem, int splits)
{
	static int cache[FM_MAX_DEVICES][9] = {};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= FM_MAX_DEVICES) { return sm_count() / splits; }
	if (cache[dev][splits] == 0)
	{
		cudaLaunchConfig_t cfg = {};
		cfg.gridDim = dim3(1, 1, (unsigned)splits);
		cfg.blockDim = dim3(FM_THREADS, 1, 1);
		cfg.dynamicSmemBytes = smem;
		cudaLaunchAttribute attr[1];
		attr[0].id = cudaLaunchAttributeClusterDimension;
		attr[0].val.clusterDim.x = 1;
		attr[0].val.clusterDim.y = 1;
		attr[0].val.clusterDim.z = (unsigned)splits;
		cfg.attrs = attr;
		cfg.numAttrs = 1;
		int n = 0;
		if (cudaOccupancyMaxActiveClusters(&n, (const void *)kern, &cfg) != cudaSuccess || n <= 0)
		{
			(void)cudaGetLastError();
			n = max(1, sm_count() / splits);
		}
		cache[dev][splits] = n;
	}
	return cache[dev][splits];
}

template <int KS, int PITCH, int PT, int CKP>
static int launch_float_map(const xnor_b200_conv_desc * desc, FloatMapParams p, cudaStream_t stream, int only_cost, double * cost)
{
	using SH = FloatMapShape<KS, PITCH, PT, CKP>;
	auto kern = float_conv_map_kernel<KS, PITCH, PT, CKP>;
	int rc = ensure_dynamic_smem((const void *)kern, SH::SMEM);
	if (rc != XNOR_B200_OK) { return rc; }
	const int HW = desc->h * desc->w;
	p.ptiles = (HW + PT - 1) / PT;
	const int mtiles = (desc->n + FM_FT - 1) / FM_FT;
	const long long tiles = (long long)p.ptiles * desc->batch * mtiles;
	if ((long long)p.ptiles * desc->batch > 0x7fffffffLL || mtiles > 65535) { return XNOR_B200_ERR_TOO_LARGE; }
	// Channel split: the one with the least (waves x work per CTA); a CTA's work is its channels times the pixel
	// slots it computes plus a staging share that does not shrink with the tile.
	int best = 1;
	double best_cost = 0.0;
	for (int s = 1; s <= 8; s *= 2)
	{
		if (desc->c % (s * SH::CK) != 0) { break; }
		const long long waves = (tiles + max_active_clusters(kern, SH::SMEM, s) - 1) / max_active_clusters(kern, SH::SMEM, s);
		const double c = (double)waves * ((double)(desc->c / s) * (PT + 64) + 4000.0 + 500.0 * s);
		if (s == 1 || c < best_cost) { best = s; best_cost = c; }
	}
	*cost = best_cost;
	if (only_cost) { return XNOR_B200_OK; }
	p.splits = best;
	p.chans_per_split = desc->c / best;

	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3((unsigned)(p.ptiles * desc->batch), (unsigned)mtiles, (unsigned)best);
	cfg.blockDim = dim3(FM_THREADS, 1, 1);
	cfg.dynamicSmemBytes = SH::SMEM;
	cfg.stream = stream;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeClusterDimension;
	attr[0].val.clusterDim.x = 1;
	attr[0].val.clusterDim.y = 1;
	attr[0].val.clusterDim.z = (unsigned)best;
	cfg.attrs = attr;
	cfg.numAttrs = 1;
	cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
	if (e != cudaSuccess) { return cuda_fail(e); }
	return check_launch();
}

// Both pixel-tile sizes are costed; the cheaper one is launched.
template <int KS, int PITCH, int CKP>
static int launch_float_map_best(const xnor_b200_conv_desc * desc, const FloatMapParams & p, cudaStream_t stream)
{
	double c96 = 0.0, c192 = 0.0;
	int rc = launch_float_map<KS, PITCH, 96, CKP>(desc, p, stream, 1, &c96);
	if (rc != XNOR_B200_OK) { return rc; }
	rc = launch_float_map<KS, PITCH, 192, CKP>(desc, p, stream, 1, &c192);
	if (rc != XNOR_B200_OK) { return rc; }
	return (c96 < c192) ? launch_float_map<KS, PITCH, 96, CKP>(desc, p, stream, 0, &c96)
	                    : launch_float_map<KS, PITCH, 192, CKP>(desc, p, stream, 0, &c192);
}

}  // namespace xnor

using namespace xnor;

extern "C" size_t xnor_b200_float_conv_map_weights_bytes(const xnor_b200_conv_desc * desc)
{
	if (desc == nullptr || validate_desc(desc) != XNOR_B200_OK || !map_conv_shape_ok(desc)) { return 0; }
	const size_t tiles = ((size_t)desc->n + FM_FT - 1) / FM_FT;
	return tiles * FM_FT * (size_t)desc->c * desc->size * desc->size * sizeof(float);
}

extern "C" int xnor_b200_float_conv_map_prepare(const xnor_b200_conv_desc * desc, const float * weights, float * blocked, void * stream)
{
	if (desc == nullptr || weights == nullptr || blocked == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (!map_conv_shape_ok(desc)) { return XNOR_B200_ERR_INVALID; }
	const int K = desc->c * desc->size * desc->size;
	const size_t total = xnor_b200_float_conv_map_weights_bytes(desc) / sizeof(float);
	const int grid = (int)min((total + 255) / 256, (size_t)sm_count() * 8);
	float_conv_map_block_weights_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(weights, blocked, desc->n, K, total);
	return check_launch();
}

extern "C" int xnor_b200_float_conv_map(const xnor_b200_conv_desc * desc, const float * input, const float * blocked_weights,
		const float * biases, float * output, void * stream)
{
	return xnor_b200_float_conv_map_yolo(desc, input, blocked_weights, biases, output, 0, stream);
}

extern "C" int xnor_b200_float_conv_map_yolo(const xnor_b200_conv_desc * desc, const float * input, const float * blocked_weights,
		const float * biases, float * output, int yolo_entries, void * stream)
{
	if (yolo_entries < 0 || (yolo_entries > 0 && (yolo_entries < 5 || desc == nullptr || desc->n % yolo_entries != 0))) { return XNOR_B200_ERR_INVALID; }
	if (desc == nullptr || input == nullptr || blocked_weights == nullptr || output == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = validate_desc(desc);
	if (rc != XNOR_B200_OK) { return rc; }
	if (!map_conv_shape_ok(desc)) { return XNOR_B200_ERR_INVALID; }
	if ((reinterpret_cast<uintptr_t>(blocked_weights) & 15) != 0) { return XNOR_B200_ERR_ALIGNMENT; }

	FloatMapParams p = {};
	p.in = input; p.wblk = blocked_weights; p.bias = biases; p.out = output;
	p.C = desc->c; p.H = desc->h; p.W = desc->w; p.N = desc->n;
	p.K = desc->c * desc->size * desc->size;
	p.leaky = (desc->activation == XNOR_B200_LEAKY) ? 1 : 0;
	p.yolo_entries = yolo_entries;
	// channels per pipeline stage: 16 for 3x3 on the small pitch when the channel count allows (half the barriers)
	if (desc->size == 1)
	{
		if (desc->c <= F1_MAX_K) { return launch_float_1x1(desc, p, (cudaStream_t)stream); }
		return launch_float_map_best<1, 16, 32>(desc, p, (cudaStream_t)stream);
	}
	if (desc->h <= 14 && desc->w <= 14)
	{
		return (desc->c % 64 == 0) ? launch_float_map_best<3, 16, 16>(desc, p, (cudaStream_t)stream)
		                           : launch_float_map_best<3, 16, 8>(desc, p, (cudaStream_t)stream);
	}
	return launch_float_map_best<3, 32, 8>(desc, p, (cudaStream_t)stream);
}
