// Headless stand-in for <opencv2/opencv.hpp>, used ONLY to compile the reference's own CPU sources as test oracles:
// the four xnor translation units (make ref) and the whole CPU library for full-network runs (build_refnet.py).
// A forward pass on a raw float tensor never calls OpenCV; the reference merely includes this header from its
// umbrella header and names OpenCV types in drawing, image-loading and heat-map code that the oracle never reaches.
// So: types with the right names and members, arithmetic on rectangles done properly (box.cpp's cv::Rect overloads
// of iou), every drawing / file / window function a no-op.  Test infrastructure: nothing in the product links this.
#pragma once
#include <math.h>
#include <cmath>
#include <cstdarg>
#include <climits>
#include <cfloat>
#include <chrono>
#include <ctime>
#include <algorithm>
#include <string>
#include <vector>

#define CV_VERSION "0.0.0-headless-stand-in"
#define CV_8UC1 0
#define CV_8UC3 16
#define CV_32FC1 5
#define CV_32FC3 21
#define CV_RGB(r, g, b) cv::Scalar((b), (g), (r), 0)

namespace cv
{
	template <typename T> struct Point_
	{
		T x = 0, y = 0;
		Point_() {}
		Point_(T a, T b) : x(a), y(b) {}
		Point_ operator+(const Point_ & o) const { return Point_(x + o.x, y + o.y); }
		Point_ operator-(const Point_ & o) const { return Point_(x - o.x, y - o.y); }
	};
	typedef Point_<int> Point;
	typedef Point_<float> Point2f;
	template <typename T> struct Size_
	{
		T width = 0, height = 0;
		Size_() {}
		Size_(T w, T h) : width(w), height(h) {}
		T area() const { return width * height; }
	};
	typedef Size_<int> Size;
	typedef Size_<float> Size2f;
	template <typename T> struct Rect_
	{
		T x = 0, y = 0, width = 0, height = 0;
		Rect_() {}
		Rect_(T x_, T y_, T w_, T h_) : x(x_), y(y_), width(w_), height(h_) {}
		T area() const { return width * height; }
		Point_<T> tl() const { return Point_<T>(x, y); }
		Point_<T> br() const { return Point_<T>(x + width, y + height); }
		bool operator==(const Rect_ & o) const { return x == o.x && y == o.y && width == o.width && height == o.height; }
		// intersection; empty when the rectangles do not overlap
		Rect_ operator&(const Rect_ & o) const
		{
			const T x1 = std::max(x, o.x), y1 = std::max(y, o.y);
			const T x2 = std::min(x + width, o.x + o.width), y2 = std::min(y + height, o.y + o.height);
			if (x2 <= x1 || y2 <= y1) { return Rect_(); }
			return Rect_(x1, y1, x2 - x1, y2 - y1);
		}
		Rect_ operator|(const Rect_ & o) const
		{
			const T x1 = std::min(x, o.x), y1 = std::min(y, o.y);
			const T x2 = std::max(x + width, o.x + o.width), y2 = std::max(y + height, o.y + o.height);
			return Rect_(x1, y1, x2 - x1, y2 - y1);
		}
	};
	typedef Rect_<int> Rect;
	typedef Rect_<float> Rect2f;
	struct Scalar
	{
		double val[4] = {0, 0, 0, 0};
		Scalar() {}
		Scalar(double a, double b = 0, double c = 0, double d = 0) { val[0] = a; val[1] = b; val[2] = c; val[3] = d; }
		double operator[](int i) const { return val[i]; }
	};
	struct MatSize { int operator[](int) const { return 0; } Size operator()() const { return Size(); } };
	// No pixel storage: every Mat is empty, which is what the image helpers see when nothing was ever loaded.
	struct Mat
	{
		int rows = 0, cols = 0, flags = 0, dims = 0;
		unsigned char * data = nullptr;
		size_t step = 0;
		MatSize size;
		Mat() {}
		Mat(int, int, int) {}
		Mat(int, int, int, const Scalar &) {}
		Mat(Size, int) {}
		Mat(Size, int, const Scalar &) {}
		Mat(int, int, int, void *, size_t = 0) {}
		int type() const { return 0; }
		int channels() const { return 0; }
		int depth() const { return 0; }
		bool empty() const { return true; }
		size_t total() const { return 0; }
		size_t elemSize() const { return 0; }
		bool isContinuous() const { return true; }
		Mat clone() const { return Mat(); }
		void copyTo(Mat &) const {}
		void copyTo(Mat &, const Mat &) const {}
		void convertTo(Mat &, int, double = 1, double = 0) const {}
		Mat rowRange(int, int) const { return Mat(); }
		Mat colRange(int, int) const { return Mat(); }
		Mat operator()(const Rect &) const { return Mat(); }
		Mat & operator=(const Scalar &) { return *this; }
		Mat & operator=(double) { return *this; }
		Mat & setTo(const Scalar &) { return *this; }
		Mat & operator+=(const Mat &) { return *this; }
		Mat & operator-=(const Mat &) { return *this; }
		Mat & operator*=(double) { return *this; }
		template <typename T> T & at(int, int) { static T dummy; return dummy; }
		template <typename T> const T & at(int, int) const { static T dummy; return dummy; }
		template <typename T> T * ptr(int = 0) { return nullptr; }
		template <typename T> const T * ptr(int = 0) const { return nullptr; }
		static Mat zeros(int, int, int) { return Mat(); }
		static Mat zeros(Size, int) { return Mat(); }
		void release() {}
	};
	inline Mat operator-(const Mat &, double) { return Mat(); }
	inline Mat operator-(const Mat &, const Mat &) { return Mat(); }
	inline Mat operator+(const Mat &, const Mat &) { return Mat(); }
	inline Mat operator*(const Mat &, double) { return Mat(); }
	inline Mat operator/(const Mat &, double) { return Mat(); }
	inline Mat operator&(const Mat &, const Mat &) { return Mat(); }
	inline Mat operator|(const Mat &, const Mat &) { return Mat(); }

	enum LineTypes { FILLED = -1, LINE_4 = 4, LINE_8 = 8, LINE_AA = 16 };
	enum HersheyFonts { FONT_HERSHEY_SIMPLEX = 0, FONT_HERSHEY_PLAIN = 1, FONT_HERSHEY_DUPLEX = 2, FONT_HERSHEY_COMPLEX = 3 };
	enum InterpolationFlags { INTER_NEAREST = 0, INTER_LINEAR = 1, INTER_CUBIC = 2, INTER_AREA = 3 };
	enum ColormapTypes { COLORMAP_AUTUMN = 0, COLORMAP_BONE = 1, COLORMAP_JET = 2, COLORMAP_HOT = 11 };
	enum ColorConversionCodes { COLOR_BGR2RGB = 4, COLOR_RGB2BGR = 4, COLOR_BGR2GRAY = 6, COLOR_GRAY2BGR = 8, COLOR_BGR2HSV = 40, COLOR_HSV2BGR = 54 };
	enum ImreadModes { IMREAD_UNCHANGED = -1, IMREAD_GRAYSCALE = 0, IMREAD_COLOR = 1 };
	enum RotateFlags { ROTATE_90_CLOCKWISE = 0, ROTATE_180 = 1, ROTATE_90_COUNTERCLOCKWISE = 2 };
	enum WindowFlags { WINDOW_NORMAL = 0, WINDOW_AUTOSIZE = 1 };

	inline int waitKey(int = 0) { return -1; }
	inline void line(Mat &, Point, Point, const Scalar &, int = 1, int = 8, int = 0) {}
	inline void rectangle(Mat &, Point, Point, const Scalar &, int = 1, int = 8, int = 0) {}
	inline void rectangle(Mat &, Rect, const Scalar &, int = 1, int = 8, int = 0) {}
	inline void circle(Mat &, Point, int, const Scalar &, int = 1, int = 8, int = 0) {}
	inline void ellipse(Mat &, Point, Size, double, double, double, const Scalar &, int = 1, int = 8, int = 0) {}
	inline int floodFill(Mat &, Point, Scalar, Rect * = nullptr, Scalar = Scalar(), Scalar = Scalar(), int = 4) { return 0; }
	inline void putText(Mat &, const std::string &, Point, int, double, Scalar, int = 1, int = 8, bool = false) {}
	inline Size getTextSize(const std::string &, int, double, int, int * baseline) { if (baseline) { *baseline = 0; } return Size(); }
	inline void cvtColor(const Mat &, Mat &, int, int = 0) {}
	inline void resize(const Mat &, Mat &, Size, double = 0, double = 0, int = 1) {}
	inline void rotate(const Mat &, Mat &, int) {}
	inline void split(const Mat &, std::vector<Mat> &) {}
	inline void merge(const std::vector<Mat> &, Mat &) {}
	inline void minMaxLoc(const Mat &, double * mn, double * mx = nullptr, Point * = nullptr, Point * = nullptr) { if (mn) { *mn = 0; } if (mx) { *mx = 0; } }
	inline Scalar mean(const Mat &) { return Scalar(); }
	inline void applyColorMap(const Mat &, Mat &, int) {}
	inline bool imwrite(const std::string &, const Mat &, const std::vector<int> & = std::vector<int>()) { return false; }
	inline Mat imread(const std::string &, int = 1) { return Mat(); }
	inline void imshow(const std::string &, const Mat &) {}
	inline void namedWindow(const std::string &, int = 1) {}
	inline void resizeWindow(const std::string &, int, int) {}
	inline void moveWindow(const std::string &, int, int) {}
	inline void destroyAllWindows() {}
	inline void destroyWindow(const std::string &) {}
	inline void setNumThreads(int) {}
}
