// Basic value types of the operator layer: algebras, enums and their string parsers, integer pairs, tensor
// shapes and the TF-style window geometry. Names and semantics follow the UpStride engine
// (src/algebras.hpp:17-27, src/backend/types.hpp:14-175, src/backend/tensor.hpp:35-276, src/utils.cc:10-50)
// so that code written against it compiles against this layer.
#pragma once

#include <algorithm>
#include <cstdint>
#include <initializer_list>
#include <ostream>
#include <stdexcept>
#include <string>
#include <vector>

namespace upstride {

enum Algebra { REAL, COMPLEX, QUATERNION, GA_300 };
static const int MULTIVECTOR_DIM[] = {1, 2, 4, 8};

enum class Padding { SAME, VALID, EXPLICIT };
enum class DataFormat { NCHW, NHWC, NC };
enum class FilterLayout { OIHW, OHWI, HWIO, IO, OI };

typedef std::vector<int32_t> IntTuple;

inline std::string upperCase(std::string s) {
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::toupper(c); });
    return s;
}

inline Padding paddingFromString(const std::string& text) {
    const std::string t = upperCase(text);
    if (t == "SAME") return Padding::SAME;
    if (t == "VALID") return Padding::VALID;
    if (t == "EXPLICIT") return Padding::EXPLICIT;
    throw std::invalid_argument("Invalid padding encountered: " + text);
}

inline DataFormat dataFormatFromString(const std::string& text) {
    const std::string t = upperCase(text);
    if (t == "NCHW") return DataFormat::NCHW;
    if (t == "NHWC") return DataFormat::NHWC;
    if (t == "NC") return DataFormat::NC;
    throw std::invalid_argument("Invalid data format encountered: " + text);
}

inline FilterLayout filterLayoutFromString(const std::string& text) {
    const std::string t = upperCase(text);
    if (t == "OIHW") return FilterLayout::OIHW;
    if (t == "OHWI") return FilterLayout::OHWI;
    if (t == "HWIO") return FilterLayout::HWIO;
    if (t == "IO") return FilterLayout::IO;
    if (t == "OI") return FilterLayout::OI;
    throw std::invalid_argument("Invalid filter layout encountered: " + text);
}

inline const char* dataFormatToString(DataFormat f) {
    return f == DataFormat::NCHW ? "NCHW" : (f == DataFormat::NHWC ? "NHWC" : "NC");
}

inline const char* filterLayoutToString(FilterLayout l) {
    switch (l) {
        case FilterLayout::OIHW: return "OIHW";
        case FilterLayout::OHWI: return "OHWI";
        case FilterLayout::HWIO: return "HWIO";
        case FilterLayout::IO: return "IO";
        case FilterLayout::OI: return "OI";
    }
    return "?";
}

// Index of the channel / height / width dimension of a 4-D activation shape.
inline int getDepthDimensionNumber(DataFormat f) { return f == DataFormat::NCHW ? 1 : 3; }
inline int getHeightDimensionNumber(DataFormat f) { return f == DataFormat::NCHW ? 2 : 1; }
inline int getWidthDimensionNumber(DataFormat f) { return f == DataFormat::NCHW ? 3 : 2; }

struct IntPair {
    int x, y;
    IntPair() : x(0), y(0) {}
    IntPair(int both) : x(both), y(both) {}
    IntPair(int x, int y) : x(x), y(y) {}
    IntPair(const IntTuple& t) {
        if (t.size() == 1) { x = y = t[0]; }
        else if (t.size() == 2) { x = t[0]; y = t[1]; }
        else throw std::invalid_argument("one or two values expected");
    }
    bool operator==(const IntPair& o) const { return x == o.x && y == o.y; }
    bool operator!=(const IntPair& o) const { return !(*this == o); }
    bool operator<(const IntPair& o) const { return x < o.x || (x == o.x && y < o.y); }
    IntPair operator+(const IntPair& o) const { return IntPair(x + o.x, y + o.y); }
    static const IntPair ZEROS, ONES;
};
inline const IntPair IntPair::ZEROS(0, 0);
inline const IntPair IntPair::ONES(1, 1);

// Reads a stride / dilation attribute given with 1, 2 or 4 entries (the 4-entry form is a full NCHW/NHWC
// vector whose batch and channel entries must equal validBatchAndChannelVal).
inline bool getSpatialStep(const IntTuple& tuple, int validBatchAndChannelVal, IntPair& result) {
    if (tuple.size() == 1) { result = IntPair(tuple[0]); return true; }
    if (tuple.size() == 2) { result = IntPair(tuple[0], tuple[1]); return true; }
    if (tuple.size() == 4) {
        result = IntPair(tuple[1], tuple[2]);
        return tuple[0] == validBatchAndChannelVal && tuple[3] == validBatchAndChannelVal;
    }
    return false;
}

// Output size and padding of a sliding window under the TensorFlow convention.
inline int computeWindowedOutputSizeAndPadding(int inputSize, int filterSize, int dilation, int stride, Padding padding,
                                               int& paddingBefore, int& paddingAfter) {
    const int effective = (filterSize - 1) * dilation + 1;
    if (padding == Padding::VALID) {
        paddingBefore = paddingAfter = 0;
        return (inputSize - effective + stride) / stride;
    }
    if (padding == Padding::SAME) {
        const int out = (inputSize + stride - 1) / stride;
        const int needed = std::max(0, (out - 1) * stride + effective - inputSize);
        paddingBefore = needed / 2;               // an odd total puts the extra pixel after
        paddingAfter = needed - paddingBefore;
        return out;
    }
    throw std::invalid_argument("Invalid padding");
}

inline int computeWindowedOutputSizeAndPadding(int inputSize, int filterSize, int dilation, int stride, int paddingBefore,
                                               int paddingAfter) {
    const int effective = (filterSize - 1) * dilation + 1;
    return (inputSize + paddingBefore + paddingAfter - effective + stride) / stride;
}

// Tensor shape: a short vector of extents with the slicing / splitting helpers the operators rely on.
class Shape {
    std::vector<int> dims;

public:
    static const Shape EMPTY;
    Shape() {}
    explicit Shape(int size) : dims((size_t)size, 0) {}
    Shape(std::initializer_list<int> l) : dims(l) {}
    Shape(int size, const int* values) : dims(values, values + size) {}
    explicit Shape(const std::vector<int>& v) : dims(v) {}

    int getSize() const { return (int)dims.size(); }
    const int* getShapePtr() const { return dims.data(); }
    int operator[](int i) const { return dims[(size_t)(i < 0 ? i + getSize() : i)]; }
    int& operator[](int i) { return dims[(size_t)(i < 0 ? i + getSize() : i)]; }

    int numel() const {
        if (dims.empty()) return 0;
        long long n = 1;
        for (int d : dims) n *= d;
        return (int)n;
    }
    // A shape with no dimensions or with a zero extent holds no data.
    bool empty() const { return numel() == 0; }

    bool operator==(const Shape& o) const { return dims == o.dims; }
    bool operator!=(const Shape& o) const { return dims != o.dims; }
    // <0, 0, >0 like strcmp: first by rank, then lexicographically.
    int compare(const Shape& o) const {
        if (getSize() != o.getSize()) return getSize() < o.getSize() ? -1 : 1;
        for (int i = 0; i < getSize(); ++i)
            if (dims[i] != o.dims[i]) return dims[i] < o.dims[i] ? -1 : 1;
        return 0;
    }

    // Sub-shape [begin, end); negative indices count from the back, end == 0 means "to the end".
    Shape slice(int begin, int end = 0) const {
        if (begin < 0) begin += getSize();
        if (end <= 0) end += getSize();
        if (begin < 0 || end > getSize() || begin > end) throw std::invalid_argument("Invalid shape slice");
        return Shape(std::vector<int>(dims.begin() + begin, dims.begin() + end));
    }
    // Shape of one of `parts` equal blocks along the outermost dimension.
    Shape split(int parts) const {
        if (dims.empty() || dims[0] % parts != 0) throw std::invalid_argument("Cannot split the outermost dimension");
        Shape s(*this);
        s.dims[0] /= parts;
        return s;
    }

    int depth(DataFormat f) const { return dims[(size_t)getDepthDimensionNumber(f)]; }
    int& depth(DataFormat f) { return dims[(size_t)getDepthDimensionNumber(f)]; }
    int height(DataFormat f) const { return dims[(size_t)getHeightDimensionNumber(f)]; }
    int& height(DataFormat f) { return dims[(size_t)getHeightDimensionNumber(f)]; }
    int width(DataFormat f) const { return dims[(size_t)getWidthDimensionNumber(f)]; }
    int& width(DataFormat f) { return dims[(size_t)getWidthDimensionNumber(f)]; }
};
inline const Shape Shape::EMPTY;

inline std::ostream& operator<<(std::ostream& os, const Shape& s) {
    os << "(";
    for (int i = 0; i < s.getSize(); ++i) os << (i ? ", " : "") << s[i];
    return os << ")";
}

}  // namespace upstride
