// Headless stand-in for <opencv2/opencv.hpp>, used ONLY to compile the reference's own
// xnor CPU sources (gemm.cpp, im2col.cpp, activations.cpp, convolutional_layer.cpp) as a
// test oracle.  The xnor forward path never calls OpenCV; the reference merely includes
// this header from its umbrella header, so empty types with the right names are enough.
// Test infrastructure: nothing in the product links against this.
#pragma once
#include <cmath>
#include <cstdarg>
#include <climits>
#include <cfloat>
#include <string>
#include <vector>

namespace cv
{
	struct Mat {};
	struct Size { int width = 0, height = 0; Size() {} Size(int w, int h) : width(w), height(h) {} };
	struct Size2f { float width = 0, height = 0; };
	struct Point { int x = 0, y = 0; Point() {} Point(int a, int b) : x(a), y(b) {} };
	struct Point2f { float x = 0, y = 0; Point2f() {} Point2f(float a, float b) : x(a), y(b) {} };
	struct Rect { int x = 0, y = 0, width = 0, height = 0; };
	struct Rect2f { float x = 0, y = 0, width = 0, height = 0; };
	struct Scalar { double val[4] = {0, 0, 0, 0}; Scalar() {} Scalar(double a, double b = 0, double c = 0, double d = 0) { val[0] = a; val[1] = b; val[2] = c; val[3] = d; } };
	enum LineTypes { FILLED = -1, LINE_4 = 4, LINE_8 = 8, LINE_AA = 16 };
	enum HersheyFonts { FONT_HERSHEY_SIMPLEX = 0, FONT_HERSHEY_PLAIN = 1 };
	enum InterpolationFlags { INTER_NEAREST = 0, INTER_LINEAR = 1, INTER_CUBIC = 2, INTER_AREA = 3 };
	enum ColormapTypes { COLORMAP_AUTUMN = 0, COLORMAP_JET = 2 };
}
