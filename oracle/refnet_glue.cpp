// Test infrastructure, not product code.
//
// Flat C wrappers around the reference's OWN network API -- load_network_custom (src-lib/weights.cpp:665-691: cfg parser,
// .weights loader, fuse_conv_batchnorm, calculate_binary_weights), network_predict_ptr (src-lib/darknet_network.cpp:813),
// get_network_boxes (:1250) and do_nms_sort (src-lib/box.cpp) -- so that the Python tests can run a whole network through
// the reference's CPU code and compare every layer and the final detections with the CUDA path.  build_refnet.py compiles
// the reference's CPU translation units unmodified from the mounted tree and links them with this file into
// oracle/_ref/liboracle_refnet.so; reference symbols that live in translation units left out of that build (windows,
// image files, charts, the command line) are bound to refnet_unreachable(), which aborts.
#include "darknet_internal.hpp"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

extern "C" void refnet_unreachable()
{
	std::fprintf(stderr, "oracle/_ref: a reference function outside the compiled subset was called\n");
	std::abort();
}

// Reference functions from left-out translation units that a load does reach, with results that cannot influence a forward
// pass: the display colour of a class (darknet_image.cpp; load_weights assigns one per class, src-lib/weights.cpp:819-823).
float Darknet::get_color(int, int, int) { return 0.0f; }

extern "C"
{

__attribute__((visibility("default"))) void * refnet_load(const char * cfg, const char * weights, int batch)
{
	return load_network_custom(cfg, weights, 0, batch);
}

__attribute__((visibility("default"))) void refnet_free(void * net)
{
	if (net) { free_network_ptr(net); }
}

__attribute__((visibility("default"))) int refnet_layers(void * ptr)
{
	return reinterpret_cast<Darknet::Network *>(ptr)->n;
}

// out[0..9] = type, outputs (per image), out_c, out_h, out_w, xnor, batch, n, activation, has align_bit_weights
__attribute__((visibility("default"))) void refnet_layer_info(void * ptr, int i, int * out)
{
	const Darknet::Layer & l = reinterpret_cast<Darknet::Network *>(ptr)->layers[i];
	out[0] = (int)l.type; out[1] = l.outputs; out[2] = l.out_c; out[3] = l.out_h; out[4] = l.out_w;
	out[5] = l.xnor; out[6] = l.batch; out[7] = l.n; out[8] = (int)l.activation; out[9] = l.align_bit_weights != nullptr;
}

__attribute__((visibility("default"))) int refnet_predict(void * ptr, float * input)
{
	return network_predict_ptr(ptr, input) != nullptr ? 0 : 1;
}

// copies batch*outputs floats of layer i's output (as left by the last predict)
__attribute__((visibility("default"))) int refnet_layer_output(void * ptr, int i, float * dst, int count)
{
	const Darknet::Layer & l = reinterpret_cast<Darknet::Network *>(ptr)->layers[i];
	if (l.output == nullptr || count > l.outputs * l.batch) { return 1; }
	std::memcpy(dst, l.output, sizeof(float) * (size_t)count);
	return 0;
}

// folded weights / biases of a convolutional layer after load (for the batch-norm fold check)
__attribute__((visibility("default"))) int refnet_layer_weights(void * ptr, int i, float * weights, int nweights, float * biases, int nbiases)
{
	const Darknet::Layer & l = reinterpret_cast<Darknet::Network *>(ptr)->layers[i];
	if (l.weights == nullptr || nweights > l.nweights || nbiases > l.n) { return 1; }
	std::memcpy(weights, l.weights, sizeof(float) * (size_t)nweights);
	std::memcpy(biases, l.biases, sizeof(float) * (size_t)nbiases);
	return 0;
}

// Detections of image 0 of the last predict: get_network_boxes + do_nms_sort.  One row per (detection, class) with a
// probability above zero after suppression: {x, y, w, h, objectness, class, probability}.  Returns the number of rows.
__attribute__((visibility("default"))) int refnet_detections(void * ptr, int w, int h, float thresh, float nms, int letter, float * rows, int max_rows)
{
	int num = 0;
	DarknetDetection * dets = get_network_boxes(ptr, w, h, thresh, 0.5f, nullptr, 1, &num, letter);
	Darknet::Network & net = *reinterpret_cast<Darknet::Network *>(ptr);
	const int classes = net.layers[net.n - 1].classes;
	if (nms > 0.0f && num > 0) { do_nms_sort(dets, num, classes, nms); }
	int count = 0;
	for (int i = 0; i < num; ++i)
	{
		for (int c = 0; c < classes; ++c)
		{
			if (dets[i].prob[c] > 0.0f && count < max_rows)
			{
				float * r = rows + 7 * count++;
				r[0] = dets[i].bbox.x; r[1] = dets[i].bbox.y; r[2] = dets[i].bbox.w; r[3] = dets[i].bbox.h;
				r[4] = dets[i].objectness; r[5] = (float)c; r[6] = dets[i].prob[c];
			}
		}
	}
	free_detections(dets, num);
	return count;
}


// do_nms_sort (src-lib/box.cpp:951) on caller-made detections: boxes [total][4], objectness [total], probs [total][classes];
// the probabilities come back in the caller's order with the suppressed ones zeroed.
__attribute__((visibility("default"))) void refnet_nms_sort(const float * boxes, const float * objectness, float * probs, int total, int classes, float thresh)
{
	std::vector<DarknetDetection> dets((size_t)total);
	std::vector<float> own((size_t)total * classes);
	std::memcpy(own.data(), probs, sizeof(float) * own.size());
	for (int i = 0; i < total; ++i)
	{
		std::memset(&dets[i], 0, sizeof(DarknetDetection));
		dets[i].bbox.x = boxes[4 * i]; dets[i].bbox.y = boxes[4 * i + 1]; dets[i].bbox.w = boxes[4 * i + 2]; dets[i].bbox.h = boxes[4 * i + 3];
		dets[i].classes = classes;
		dets[i].objectness = objectness[i];
		dets[i].prob = own.data() + (size_t)i * classes;
		dets[i].track_id = i;
	}
	do_nms_sort(dets.data(), total, classes, thresh);
	for (int i = 0; i < total; ++i)
	{
		std::memcpy(probs + (size_t)dets[i].track_id * classes, dets[i].prob, sizeof(float) * classes);
	}
}

}
