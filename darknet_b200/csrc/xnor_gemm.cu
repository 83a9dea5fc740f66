// XNOR-popcount GEMM with the per-filter mean scale, bias, leaky/linear activation and optional
// shortcut add fused into the epilogue.
//
// Replaces gemm_nn_custom_bin_mean_transposed_gpu (src-lib/im2col_kernels.cu:793-956, :1156-1193; a wmma
// b1 kernel that reads both operands straight from global memory, one warp per 8x16 outputs) and, on the
// CPU side, gemm_nn_custom_bin_mean_transposed + add_bias + leaky (src-lib/gemm.cpp:907-1019,
// src-lib/convolutional_layer.cpp:1269-1289, src-lib/gemm.cpp:1472-1498).
//
// Operands: A [M][lda_words] and B [n_total][ldb_words] 32-bit words, K bits of data per row followed by
// zero bits.  With zero padding on both sides  popc(a ^ b)  over whole words counts exactly the
// disagreeing bits among the first K, so   2*count - K  =  K - 2*sum popc(a ^ b)   with no padding
// correction term (the reference subtracts f1 because its A padding is complemented).
//
// Tiling: a CTA computes a BM x BN tile; operands are staged through a STAGES-deep cp.async ring in shared
// memory (row pitch KT+4 words so that 16-byte reads of 8 consecutive rows hit 32 distinct banks); every
// thread owns a TM x TN register tile of int32 accumulators and consumes four K-words per 16-byte shared
// load.  Accumulators are exact integers; the epilogue mirrors the reference CPU rounding order: one
// fp32 multiply, one fp32 add, then the leaky blend -- never a fused multiply-add.
#include "xnor_common.cuh"

namespace xnor
{

struct GemmParams
{
	const uint32_t * A;
	const uint32_t * B;
	int M, n_total, n_per_image, K;
	int lda_words, ldb_words;
	int kw;                 // K-words to visit, multiple of 4 (<= lda_words, ldb_words)
	float * C;
	int ldc;
	const float * mean_arr;
	const float * bias;
	int leaky;
	const float * shortcut_in;
	float * shortcut_out;
	int32_t * counts;       // when set: write integer agreement counts [M][n_total] instead of C
	int tiles_m, tiles_n;
};

__device__ __forceinline__ void cp_async_16(uint32_t * smem_dst, const uint32_t * gmem_src, bool valid)
{
	const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
	const int src_bytes = valid ? 16 : 0;   // 0 -> the 16 destination bytes are zero-filled
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

template <int BM, int BN, int TM, int TN, int KT, int STAGES>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
xnor_gemm_kernel(const GemmParams p)
{
	constexpr int TX = BN / TN;
	constexpr int TY = BM / TM;
	constexpr int NT = TX * TY;
	constexpr int PITCH = KT + 4;               // words
	constexpr int A_STAGE = BM * PITCH;
	constexpr int B_STAGE = BN * PITCH;
	constexpr int CHUNKS_ROW = KT / 4;          // 16-byte chunks per staged row
	static_assert(KT % 4 == 0, "KT must be a multiple of 4 words");

	extern __shared__ __align__(16) uint32_t smem[];
	uint32_t * sA = smem;
	uint32_t * sB = smem + STAGES * A_STAGE;

	// Tiles that share a B tile are adjacent in launch order, so concurrently running CTAs re-use the
	// same packed-activation rows out of L2 while A (small) stays resident.
	const int tile_m = blockIdx.x % p.tiles_m;
	const int tile_n = blockIdx.x / p.tiles_m;
	const int m0 = tile_m * BM;
	const int n0 = tile_n * BN;
	const int tx = threadIdx.x % TX;
	const int ty = threadIdx.x / TX;

	auto load_stage = [&](int stage, int k0)
	{
		uint32_t * dA = sA + stage * A_STAGE;
		uint32_t * dB = sB + stage * B_STAGE;
		for (int ch = threadIdx.x; ch < BM * CHUNKS_ROW; ch += NT)
		{
			const int r = ch / CHUNKS_ROW;
			const int kc = (ch - r * CHUNKS_ROW) * 4;
			if (k0 + kc >= p.kw) { continue; }          // never read by the compute loop
			const bool ok = (m0 + r < p.M);
			const uint32_t * src = ok ? p.A + (size_t)(m0 + r) * p.lda_words + k0 + kc : p.A;
			cp_async_16(dA + r * PITCH + kc, src, ok);
		}
		for (int ch = threadIdx.x; ch < BN * CHUNKS_ROW; ch += NT)
		{
			const int r = ch / CHUNKS_ROW;
			const int kc = (ch - r * CHUNKS_ROW) * 4;
			if (k0 + kc >= p.kw) { continue; }
			const bool ok = (n0 + r < p.n_total);
			const uint32_t * src = ok ? p.B + (size_t)(n0 + r) * p.ldb_words + k0 + kc : p.B;
			cp_async_16(dB + r * PITCH + kc, src, ok);
		}
	};

	int acc[TM][TN];
	#pragma unroll
	for (int i = 0; i < TM; ++i)
	{
		#pragma unroll
		for (int j = 0; j < TN; ++j) { acc[i][j] = 0; }
	}

	const int num_kt = (p.kw + KT - 1) / KT;
	#pragma unroll
	for (int s = 0; s < STAGES - 1; ++s)
	{
		if (s < num_kt) { load_stage(s, s * KT); }
		cp_async_commit();
	}

	for (int kt = 0; kt < num_kt; ++kt)
	{
		cp_async_wait<STAGES - 2>();
		__syncthreads();
		{
			const int nk = kt + STAGES - 1;
			if (nk < num_kt) { load_stage(nk % STAGES, nk * KT); }
			cp_async_commit();
		}
		const uint32_t * cA = sA + (kt % STAGES) * A_STAGE + ty * PITCH;
		const uint32_t * cB = sB + (kt % STAGES) * B_STAGE + tx * PITCH;
		auto step = [&](int k4)
		{
			uint4 a[TM], b[TN];
			#pragma unroll
			for (int i = 0; i < TM; ++i) { a[i] = *reinterpret_cast<const uint4 *>(cA + i * TY * PITCH + k4); }
			#pragma unroll
			for (int j = 0; j < TN; ++j) { b[j] = *reinterpret_cast<const uint4 *>(cB + j * TX * PITCH + k4); }
			#pragma unroll
			for (int i = 0; i < TM; ++i)
			{
				#pragma unroll
				for (int j = 0; j < TN; ++j)
				{
					acc[i][j] += __popc(a[i].x ^ b[j].x) + __popc(a[i].y ^ b[j].y)
							+ __popc(a[i].z ^ b[j].z) + __popc(a[i].w ^ b[j].w);
				}
			}
		};
		const int kvalid = min(KT, p.kw - kt * KT);   // the last stage of a short K holds fewer words
		if (kvalid == KT)
		{
			#pragma unroll
			for (int k4 = 0; k4 < KT; k4 += 4) { step(k4); }
		}
		else
		{
			for (int k4 = 0; k4 < kvalid; k4 += 4) { step(k4); }
		}
	}
	cp_async_wait<0>();

	// epilogue
	#pragma unroll
	for (int j = 0; j < TN; ++j)
	{
		const int col = n0 + j * TX + tx;
		if (col >= p.n_total) { continue; }
		const int img = col / p.n_per_image;
		const int pix = col - img * p.n_per_image;
		#pragma unroll
		for (int i = 0; i < TM; ++i)
		{
			const int m = m0 + i * TY + ty;
			if (m >= p.M) { continue; }
			if (p.counts != nullptr)
			{
				p.counts[(size_t)m * p.n_total + col] = p.K - acc[i][j];
				continue;
			}
			const size_t idx = ((size_t)img * p.M + m) * p.ldc + pix;
			const float dot = (float)(p.K - 2 * acc[i][j]);
			float v = __fmul_rn(dot, __ldg(p.mean_arr + m));
			if (p.bias != nullptr) { v = __fadd_rn(v, __ldg(p.bias + m)); }
			if (p.leaky) { v = (v < 0.0f) ? __fmul_rn(v, 0.1f) : v; }
			p.C[idx] = v;
			if (p.shortcut_out != nullptr) { p.shortcut_out[idx] = __fadd_rn(__ldg(p.shortcut_in + idx), v); }
		}
	}
}

template <int BM, int BN, int TM, int TN, int KT, int STAGES>
static int launch_config(GemmParams & p, cudaStream_t stream)
{
	constexpr int NT = (BM / TM) * (BN / TN);
	constexpr size_t SMEM = (size_t)STAGES * (BM + BN) * (KT + 4) * 4;
	auto kern = xnor_gemm_kernel<BM, BN, TM, TN, KT, STAGES>;
	int rc = ensure_dynamic_smem((const void *)kern, SMEM);
	if (rc != XNOR_B200_OK) { return rc; }
	p.tiles_m = (p.M + BM - 1) / BM;
	p.tiles_n = (p.n_total + BN - 1) / BN;
	const long long grid = (long long)p.tiles_m * p.tiles_n;
	if (grid > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	kern<<<(unsigned)grid, NT, SMEM, stream>>>(p);
	return check_launch();
}

int launch_xnor_gemm(int M, int n_total, int n_per_image, int K,
		const uint32_t * A, int lda_words, const uint32_t * B, int ldb_words,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky,
		const float * shortcut_in, float * shortcut_out, int32_t * counts, cudaStream_t stream)
{
	GemmParams p;
	p.A = A; p.B = B;
	p.M = M; p.n_total = n_total; p.n_per_image = n_per_image; p.K = K;
	p.lda_words = lda_words; p.ldb_words = ldb_words;
	p.kw = (int)round_up((size_t)(K + 31) / 32, 4);
	p.C = C; p.ldc = ldc; p.mean_arr = mean_arr; p.bias = bias; p.leaky = leaky;
	p.shortcut_in = shortcut_in; p.shortcut_out = shortcut_out; p.counts = counts;

	// Pick the largest tile that still yields at least one CTA per SM; small problems fall through to
	// the smallest tile so that batch-1 tail layers (N = 169) spread over more SMs.
	const int sms = sm_count();
	auto tiles = [&](int bm, int bn) { return (long long)((M + bm - 1) / bm) * ((n_total + bn - 1) / bn); };
	if (M > 64 && tiles(128, 128) >= sms) { return launch_config<128, 128, 8, 8, 32, 3>(p, stream); }
	if (M > 32 && tiles(64, 128) >= sms)  { return launch_config<64, 128, 4, 8, 32, 3>(p, stream); }
	if (M <= 32 && tiles(32, 256) >= sms) { return launch_config<32, 256, 4, 8, 32, 3>(p, stream); }
	if (tiles(64, 64) >= sms)             { return launch_config<64, 64, 4, 4, 32, 3>(p, stream); }
	return launch_config<32, 32, 2, 4, 32, 3>(p, stream);
}

}  // namespace xnor

using namespace xnor;

static int check_gemm_args(int M, int N, int K, const void * A, int lda, const void * B, int ldb)
{
	if (A == nullptr || B == nullptr) { return XNOR_B200_ERR_NULL; }
	if (M <= 0 || N <= 0 || K <= 0) { return XNOR_B200_ERR_INVALID; }
	if (lda < K || ldb < K || lda % 128 != 0 || ldb % 128 != 0) { return XNOR_B200_ERR_INVALID; }
	if ((((uintptr_t)A) & 15u) != 0 || (((uintptr_t)B) & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	return XNOR_B200_OK;
}

extern "C" int xnor_b200_gemm_bin_mean_transposed(int M, int N, int K,
		const uint8_t * A, int lda, const uint8_t * B, int ldb,
		float * C, int ldc, const float * mean_arr, const float * bias, int leaky_activation,
		const float * shortcut_in, float * shortcut_out, void * stream)
{
	int rc = check_gemm_args(M, N, K, A, lda, B, ldb);
	if (rc != XNOR_B200_OK) { return rc; }
	if (C == nullptr || mean_arr == nullptr) { return XNOR_B200_ERR_NULL; }
	if (ldc < N) { return XNOR_B200_ERR_INVALID; }
	if (shortcut_out != nullptr && shortcut_in == nullptr) { return XNOR_B200_ERR_NULL; }
	return launch_xnor_gemm(M, N, N, K, (const uint32_t *)A, lda / 32, (const uint32_t *)B, ldb / 32,
			C, ldc, mean_arr, bias, leaky_activation, shortcut_in, shortcut_out, nullptr, (cudaStream_t)stream);
}

extern "C" int xnor_b200_gemm_counts(int M, int N, int K, const uint8_t * A, int lda, const uint8_t * B, int ldb,
		int32_t * counts, void * stream)
{
	int rc = check_gemm_args(M, N, K, A, lda, B, ldb);
	if (rc != XNOR_B200_OK) { return rc; }
	if (counts == nullptr) { return XNOR_B200_ERR_NULL; }
	return launch_xnor_gemm(M, N, N, K, (const uint32_t *)A, lda / 32, (const uint32_t *)B, ldb / 32,
			nullptr, N, nullptr, nullptr, 0, nullptr, nullptr, counts, (cudaStream_t)stream);
}
