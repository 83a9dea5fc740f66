// Detection heads on the device: what Darknet does on the host after every forward of a [yolo] network.
//
//   xnor_b200_yolo_detections   get_yolo_detections + get_yolo_box + correct_yolo_boxes
//                               (src-lib/yolo_layer.cpp:1306-1348, :22-42, :1161-1222): every (cell, anchor) whose objectness
//                               exceeds the threshold becomes a detection -- box, objectness, objectness * class
//                               probability per class (0 where not above the threshold) -- stored in the reference's scan
//                               order (cells outer, anchors inner), the heads of a network one after the other;
//   xnor_b200_nms_sort          do_nms_sort (src-lib/box.cpp:951-1003) with box_iou (:310-344): per class, detections sorted by
//                               that class's probability, a kept detection zeroes the probability of every later one
//                               whose IoU with it exceeds the threshold;
//   xnor_b200_detection_rows    the surviving (detection, class) pairs as rows {x, y, w, h, objectness, class, probability}:
//                               the compact result a host copies back instead of the whole head tensors (Darknet pulls
//                               batch * outputs floats per head and walks them on the CPU).
//
// All three run on the caller's stream, allocate nothing and synchronise nothing; counts live in device memory, so a head can
// be appended behind another without the host knowing how many detections the first one found.
#include "xnor_common.cuh"

namespace xnor
{

constexpr int DET_THREADS = 256;
constexpr int DET_MAX_ANCHORS = 16;

struct YoloParams
{
	const float * head;          // [batch][n][4 + 1 + classes][lh * lw], activated (xnor_b200_yolo_activate)
	int batch, lw, lh, n, classes;
	float anchor_w[DET_MAX_ANCHORS], anchor_h[DET_MAX_ANCHORS];      // biases[2 * mask[a]], biases[2 * mask[a] + 1]
	int netw, neth, img_w, img_h;
	float thresh;
	int relative, letter, new_coords, append;
	float * boxes;               // [batch][max_dets][4]
	float * objectness;          // [batch][max_dets]
	float * probs;               // [batch][max_dets][classes]
	int * count;                 // [batch]: detections found so far (may exceed max_dets: the surplus is not stored)
	int max_dets;
};

// Exclusive prefix sum of one flag per thread over the CTA; returns this thread's offset, *total = number of set flags.
__device__ __forceinline__ int block_scan_flags(bool flag, int * s_warp, int * total)
{
	const int lane = threadIdx.x & 31;
	const int warp = threadIdx.x >> 5;
	const unsigned ballot = __ballot_sync(0xffffffffu, flag);
	const int in_warp = __popc(ballot & ((1u << lane) - 1u));
	if (lane == 0) { s_warp[warp] = __popc(ballot); }
	__syncthreads();
	int before = 0, all = 0;
	#pragma unroll
	for (int w = 0; w < DET_THREADS / 32; ++w)
	{
		const int c = s_warp[w];
		if (w < warp) { before += c; }
		all += c;
	}
	__syncthreads();
	*total = all;
	return before + in_warp;
}

__global__ void __launch_bounds__(DET_THREADS)
yolo_detections_kernel(const YoloParams p)
{
	__shared__ int s_warp[DET_THREADS / 32];
	const int b = blockIdx.x;
	const int cells = p.lw * p.lh;
	const int entries = 4 + 1 + p.classes;
	const float * pred = p.head + (size_t)b * p.n * entries * cells;
	int base = p.append ? p.count[b] : 0;
	__syncthreads();                                             // every thread has read the count before thread 0 rewrites it

	// correct_yolo_boxes: the network-to-image mapping, in double as the reference computes it
	int new_w = p.netw, new_h = p.neth;
	if (p.letter)
	{
		if (((float)p.netw / p.img_w) < ((float)p.neth / p.img_h)) { new_w = p.netw; new_h = (p.img_h * p.netw) / p.img_w; }
		else { new_h = p.neth; new_w = (p.img_w * p.neth) / p.img_h; }
	}
	const float deltaw = (float)(p.netw - new_w), deltah = (float)(p.neth - new_h);
	const float ratiow = (float)new_w / p.netw, ratioh = (float)new_h / p.neth;

	const int candidates = cells * p.n;
	for (int q0 = 0; q0 < candidates; q0 += DET_THREADS)
	{
		const int q = q0 + threadIdx.x;                          // reference order: cell outer, anchor inner
		const int i = q / p.n;
		const int a = q - i * p.n;
		float obj = 0.0f;
		bool hit = false;
		if (q < candidates)
		{
			obj = pred[(size_t)(a * entries + 4) * cells + i];
			hit = obj > p.thresh;
		}
		int total;
		const int slot = base + block_scan_flags(hit, s_warp, &total);
		if (hit && slot < p.max_dets)
		{
			const int row = i / p.lw, col = i - row * p.lw;
			const float * e = pred + (size_t)a * entries * cells + i;
			float bx = ((float)col + e[0]) / (float)p.lw;
			float by = ((float)row + e[(size_t)cells]) / (float)p.lh;
			float bw, bh;
			if (p.new_coords)
			{
				const float tw = e[(size_t)2 * cells], th = e[(size_t)3 * cells];
				bw = __fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(tw, tw), 4.0f), p.anchor_w[a]), (float)p.netw);
				bh = __fdiv_rn(__fmul_rn(__fmul_rn(__fmul_rn(th, th), 4.0f), p.anchor_h[a]), (float)p.neth);
			}
			else
			{
				bw = __fdiv_rn(__fmul_rn(expf(e[(size_t)2 * cells]), p.anchor_w[a]), (float)p.netw);
				bh = __fdiv_rn(__fmul_rn(expf(e[(size_t)3 * cells]), p.anchor_h[a]), (float)p.neth);
			}
			bx = (float)(((double)bx - (double)deltaw / 2. / p.netw) / (double)ratiow);
			by = (float)(((double)by - (double)deltah / 2. / p.neth) / (double)ratioh);
			bw = __fmul_rn(bw, __fdiv_rn(1.0f, ratiow));
			bh = __fmul_rn(bh, __fdiv_rn(1.0f, ratioh));
			if (!p.relative)
			{
				bx = __fmul_rn(bx, (float)p.img_w); bw = __fmul_rn(bw, (float)p.img_w);
				by = __fmul_rn(by, (float)p.img_h); bh = __fmul_rn(bh, (float)p.img_h);
			}
			const size_t d = (size_t)b * p.max_dets + slot;
			p.boxes[d * 4 + 0] = bx; p.boxes[d * 4 + 1] = by; p.boxes[d * 4 + 2] = bw; p.boxes[d * 4 + 3] = bh;
			p.objectness[d] = obj;
			for (int j = 0; j < p.classes; ++j)
			{
				const float prob = __fmul_rn(obj, e[(size_t)(5 + j) * cells]);
				p.probs[d * p.classes + j] = (prob > p.thresh) ? prob : 0.0f;
			}
		}
		base += total;
	}
	if (threadIdx.x == 0) { p.count[b] = base; }
}

// box_iou of src-lib/box.cpp:68-113, :310-344, operation for operation (no contraction into FMAs)
__device__ __forceinline__ float overlap_1d(float x1, float w1, float x2, float w2)
{
	const float l1 = __fsub_rn(x1, __fdiv_rn(w1, 2.0f)), l2 = __fsub_rn(x2, __fdiv_rn(w2, 2.0f));
	const float r1 = __fadd_rn(x1, __fdiv_rn(w1, 2.0f)), r2 = __fadd_rn(x2, __fdiv_rn(w2, 2.0f));
	return __fsub_rn(fminf(r1, r2), fmaxf(l1, l2));
}

__device__ __forceinline__ float box_iou_dev(const float4 a, const float4 b)
{
	const float w = overlap_1d(a.x, a.z, b.x, b.z);
	if (w <= 0.0f) { return 0.0f; }
	const float h = overlap_1d(a.y, a.w, b.y, b.w);
	if (h <= 0.0f) { return 0.0f; }
	const float inter = __fmul_rn(w, h);
	if (inter == 0.0f) { return 0.0f; }
	const float uni = __fsub_rn(__fadd_rn(__fmul_rn(a.z, a.w), __fmul_rn(b.z, b.w)), inter);
	return __fdiv_rn(inter, uni);
}

struct NmsParams
{
	const float * boxes;
	float * probs;
	const int * count;
	int max_dets, classes;
	float thresh;
};

// One CTA per (class, image).  Shared: candidate index, score, sorted order, alive flag per stored detection.
__global__ void __launch_bounds__(DET_THREADS)
nms_sort_kernel(const NmsParams p)
{
	extern __shared__ int s_nms[];
	const int k = blockIdx.x;
	const int b = blockIdx.y;
	const int n = min(p.count[b], p.max_dets);
	int * s_idx = s_nms;                                          // candidates of this class in storage order
	float * s_score = reinterpret_cast<float *>(s_nms + p.max_dets);
	int * s_order = s_nms + 2 * p.max_dets;                       // candidate (position in s_idx) at each rank
	int * s_alive = s_nms + 3 * p.max_dets;
	__shared__ int s_warp[DET_THREADS / 32];
	__shared__ int s_m;
	float * probs = p.probs + (size_t)b * p.max_dets * p.classes;
	const float4 * boxes = reinterpret_cast<const float4 *>(p.boxes) + (size_t)b * p.max_dets;

	// candidates: detections whose probability for this class is above zero, in storage order
	int m = 0;
	for (int d0 = 0; d0 < n; d0 += DET_THREADS)
	{
		const int d = d0 + threadIdx.x;
		const float s = (d < n) ? probs[(size_t)d * p.classes + k] : 0.0f;
		int total;
		const int slot = m + block_scan_flags(s > 0.0f, s_warp, &total);
		if (s > 0.0f) { s_idx[slot] = d; s_score[slot] = s; }
		m += total;
	}
	if (threadIdx.x == 0) { s_m = m; }
	__syncthreads();
	m = s_m;
	if (m <= 1) { return; }
	// rank by score, highest first; equal scores keep their storage order
	for (int c = threadIdx.x; c < m; c += DET_THREADS)
	{
		const float s = s_score[c];
		int rank = 0;
		for (int o = 0; o < m; ++o)
		{
			const float t = s_score[o];
			rank += (t > s || (t == s && o < c)) ? 1 : 0;
		}
		s_order[rank] = c;
		s_alive[c] = 1;
	}
	__syncthreads();
	// greedy suppression in rank order: a kept detection removes every later one that overlaps it too much
	for (int r = 0; r < m - 1; ++r)
	{
		const int ci = s_order[r];
		if (s_alive[ci])                                          // uniform: every thread reads the same flag
		{
			const float4 a = boxes[s_idx[ci]];
			for (int r2 = r + 1 + threadIdx.x; r2 < m; r2 += DET_THREADS)
			{
				const int cj = s_order[r2];
				if (s_alive[cj] && box_iou_dev(a, boxes[s_idx[cj]]) > p.thresh)
				{
					s_alive[cj] = 0;
					probs[(size_t)s_idx[cj] * p.classes + k] = 0.0f;
				}
			}
		}
		__syncthreads();
	}
}

struct RowsParams
{
	const float * boxes;
	const float * objectness;
	const float * probs;
	const int * count;
	int max_dets, classes;
	float * rows;                // [batch][max_rows][7]
	int * row_count;             // [batch]: pairs found (may exceed max_rows: the surplus is not stored)
	int max_rows;
};

__global__ void __launch_bounds__(DET_THREADS)
detection_rows_kernel(const RowsParams p)
{
	__shared__ int s_warp[DET_THREADS / 32];
	const int b = blockIdx.x;
	const int n = min(p.count[b], p.max_dets);
	const long long items = (long long)n * p.classes;
	const float * probs = p.probs + (size_t)b * p.max_dets * p.classes;
	int base = 0;
	for (long long q0 = 0; q0 < items; q0 += DET_THREADS)
	{
		const long long q = q0 + threadIdx.x;                     // (detection, class), detection-major
		const float s = (q < items) ? probs[q] : 0.0f;
		int total;
		const int slot = base + block_scan_flags(s > 0.0f, s_warp, &total);
		if (s > 0.0f && slot < p.max_rows)
		{
			const int d = (int)(q / p.classes);
			const int k = (int)(q - (long long)d * p.classes);
			const size_t dd = (size_t)b * p.max_dets + d;
			float * r = p.rows + ((size_t)b * p.max_rows + slot) * 7;
			r[0] = p.boxes[dd * 4 + 0]; r[1] = p.boxes[dd * 4 + 1]; r[2] = p.boxes[dd * 4 + 2]; r[3] = p.boxes[dd * 4 + 3];
			r[4] = p.objectness[dd]; r[5] = (float)k; r[6] = s;
		}
		base += total;
	}
	if (threadIdx.x == 0) { p.row_count[b] = base; }
}

static int check_dets(const xnor_b200_detections * d, int batch)
{
	if (d == nullptr || d->boxes == nullptr || d->objectness == nullptr || d->probs == nullptr || d->count == nullptr) { return XNOR_B200_ERR_NULL; }
	if (batch <= 0 || d->classes <= 0 || d->max_dets <= 0) { return XNOR_B200_ERR_INVALID; }
	if (d->max_dets > XNOR_B200_MAX_DETECTIONS) { return XNOR_B200_ERR_TOO_LARGE; }
	if ((((uintptr_t)d->boxes) & 15u) != 0) { return XNOR_B200_ERR_ALIGNMENT; }
	return XNOR_B200_OK;
}

}  // namespace xnor

using namespace xnor;

extern "C" int xnor_b200_yolo_detections(const xnor_b200_yolo_head * head, int batch, int netw, int neth, int img_w, int img_h,
		float thresh, int relative, int letter, int append, const xnor_b200_detections * dets, void * stream)
{
	if (head == nullptr || head->output == nullptr) { return XNOR_B200_ERR_NULL; }
	int rc = check_dets(dets, batch);
	if (rc != XNOR_B200_OK) { return rc; }
	if (head->w <= 0 || head->h <= 0 || head->n <= 0 || head->n > DET_MAX_ANCHORS || head->classes != dets->classes) { return XNOR_B200_ERR_INVALID; }
	if (netw <= 0 || neth <= 0 || img_w <= 0 || img_h <= 0) { return XNOR_B200_ERR_INVALID; }
	if ((long long)head->w * head->h * head->n > 0x7fffffffLL) { return XNOR_B200_ERR_TOO_LARGE; }
	YoloParams p;
	p.head = head->output;
	p.batch = batch; p.lw = head->w; p.lh = head->h; p.n = head->n; p.classes = head->classes;
	for (int a = 0; a < DET_MAX_ANCHORS; ++a)
	{
		p.anchor_w[a] = (a < head->n) ? head->anchors[2 * a] : 0.0f;
		p.anchor_h[a] = (a < head->n) ? head->anchors[2 * a + 1] : 0.0f;
	}
	p.netw = netw; p.neth = neth; p.img_w = img_w; p.img_h = img_h;
	p.thresh = thresh; p.relative = relative; p.letter = letter; p.new_coords = head->new_coords; p.append = append;
	p.boxes = dets->boxes; p.objectness = dets->objectness; p.probs = dets->probs; p.count = dets->count; p.max_dets = dets->max_dets;
	yolo_detections_kernel<<<batch, DET_THREADS, 0, (cudaStream_t)stream>>>(p);
	return check_launch();
}

extern "C" int xnor_b200_nms_sort(const xnor_b200_detections * dets, int batch, float nms_thresh, void * stream)
{
	int rc = check_dets(dets, batch);
	if (rc != XNOR_B200_OK) { return rc; }
	if (batch > 65535) { return XNOR_B200_ERR_TOO_LARGE; }
	NmsParams p;
	p.boxes = dets->boxes; p.probs = dets->probs; p.count = dets->count;
	p.max_dets = dets->max_dets; p.classes = dets->classes; p.thresh = nms_thresh;
	const size_t smem = (size_t)dets->max_dets * 4 * sizeof(int);
	rc = ensure_dynamic_smem((const void *)nms_sort_kernel, smem);
	if (rc != XNOR_B200_OK) { return rc; }
	nms_sort_kernel<<<dim3((unsigned)dets->classes, (unsigned)batch, 1), DET_THREADS, smem, (cudaStream_t)stream>>>(p);
	return check_launch();
}

extern "C" int xnor_b200_detection_rows(const xnor_b200_detections * dets, int batch, float * rows, int max_rows, int * row_count, void * stream)
{
	int rc = check_dets(dets, batch);
	if (rc != XNOR_B200_OK) { return rc; }
	if (rows == nullptr || row_count == nullptr) { return XNOR_B200_ERR_NULL; }
	if (max_rows <= 0) { return XNOR_B200_ERR_INVALID; }
	RowsParams p;
	p.boxes = dets->boxes; p.objectness = dets->objectness; p.probs = dets->probs; p.count = dets->count;
	p.max_dets = dets->max_dets; p.classes = dets->classes;
	p.rows = rows; p.row_count = row_count; p.max_rows = max_rows;
	detection_rows_kernel<<<batch, DET_THREADS, 0, (cudaStream_t)stream>>>(p);
	return check_launch();
}
