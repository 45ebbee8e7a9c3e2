// Operation descriptors of the operator layer. Constructor signatures, accessors, shape checks and padding
// rules follow upstride::Conv2D{,Fwd,Bwd}Descriptor (src/backend/conv2d_descriptor.hpp:113-423) and
// upstride::Dense{,Fwd,Bwd}Descriptor (src/backend/dense_descriptor.hpp:11-131). Unlike the reference,
// the ordering used as cache key is a strict weak order over every field (the reference ignores the
// filter layout and mis-orders the dense bias flag).
#pragma once

#include <sstream>
#include <tuple>

#include "types.hpp"

namespace upstride {

// Where the out-channel / in-channel / height / width extents sit in a filter shape.
class Conv2DFilterLayout {
    int o, i, h, w;

public:
    Conv2DFilterLayout(FilterLayout layout, Algebra algebra) {
        const int shift = algebra == Algebra::REAL ? 0 : 1;   // leading multivector dimension
        switch (layout) {
            case FilterLayout::OIHW: o = 0; i = 1; h = 2; w = 3; break;
            case FilterLayout::OHWI: o = 0; h = 1; w = 2; i = 3; break;
            case FilterLayout::HWIO: h = 0; w = 1; i = 2; o = 3; break;
            default: throw std::invalid_argument("Invalid filter layout for a convolution");
        }
        o += shift; i += shift; h += shift; w += shift;
    }
    int numOutputChannels(const Shape& s) const { return s[o]; }
    int numInputChannels(const Shape& s) const { return s[i]; }
    int height(const Shape& s) const { return s[h]; }
    int width(const Shape& s) const { return s[w]; }
};

class Conv2DDescriptor {
protected:
    Shape inputShape, filterShape;
    IntPair stride, dilation;
    int groups;
    Algebra algebra;
    DataFormat dataFormat;
    FilterLayout filterLayout;
    bool realValuedInput;
    IntPair padBefore, padAfter;

    auto key() const {
        return std::make_tuple(std::vector<int>(inputShape.getShapePtr(), inputShape.getShapePtr() + inputShape.getSize()),
                               std::vector<int>(filterShape.getShapePtr(), filterShape.getShapePtr() + filterShape.getSize()),
                               stride.x, stride.y, dilation.x, dilation.y, groups, (int)algebra, (int)dataFormat, (int)filterLayout,
                               realValuedInput, padBefore.x, padBefore.y, padAfter.x, padAfter.y);
    }

public:
    Conv2DDescriptor(const Shape& inputShape, const Shape& filterShape, IntPair stride, IntPair dilation, Padding paddingPreset,
                     const IntTuple& explicitPadding, int groups, Algebra algebra, DataFormat dataFormat,
                     FilterLayout filterLayout, bool realValuedInput = false)
        : inputShape(inputShape), filterShape(filterShape), stride(stride), dilation(dilation), groups(groups), algebra(algebra),
          dataFormat(dataFormat), filterLayout(filterLayout), realValuedInput(realValuedInput) {
        if (inputShape.getSize() != 4) throw std::invalid_argument("Four-dimensional input tensor expected");
        if (algebra != Algebra::REAL) {
            if (filterShape.getSize() != 5) throw std::invalid_argument("Five-dimensional filter tensor expected");
            if (filterShape[0] != MULTIVECTOR_DIM[algebra])
                throw std::invalid_argument("First filter dimension mismatch, got " + std::to_string(filterShape[0]));
        } else if (filterShape.getSize() != 4)
            throw std::invalid_argument("Four-dimensional filter tensor expected");

        const Conv2DFilterLayout filter(filterLayout, algebra);
        if (paddingPreset == Padding::EXPLICIT) {
            if (explicitPadding.size() != 4) throw std::invalid_argument("Explicit padding needs four values");
            padBefore = IntPair(explicitPadding[0], explicitPadding[1]);
            padAfter = IntPair(explicitPadding[2], explicitPadding[3]);
        } else {
            computeWindowedOutputSizeAndPadding(inputShape.height(dataFormat), filter.height(filterShape), dilation.x, stride.x,
                                                paddingPreset, padBefore.x, padAfter.x);
            computeWindowedOutputSizeAndPadding(inputShape.width(dataFormat), filter.width(filterShape), dilation.y, stride.y,
                                                paddingPreset, padBefore.y, padAfter.y);
        }
    }

    Shape getOutputShape() const {
        const Conv2DFilterLayout filter(filterLayout, algebra);
        Shape out(4);
        out[0] = inputShape[0];
        out.depth(dataFormat) = filter.numOutputChannels(filterShape);
        out.height(dataFormat) = computeWindowedOutputSizeAndPadding(inputShape.height(dataFormat), filter.height(filterShape),
                                                                     dilation.x, stride.x, padBefore.x, padAfter.x);
        out.width(dataFormat) = computeWindowedOutputSizeAndPadding(inputShape.width(dataFormat), filter.width(filterShape),
                                                                    dilation.y, stride.y, padBefore.y, padAfter.y);
        if (realValuedInput) out[0] *= MULTIVECTOR_DIM[algebra];   // a real input yields a full multivector output
        return out;
    }

    std::string toString() const {
        std::ostringstream s;
        s << inputShape << "x" << filterShape << " " << dataFormatToString(dataFormat) << " " << filterLayoutToString(filterLayout);
        if (algebra != Algebra::REAL) s << ", type " << (int)algebra;
        if (stride != IntPair::ONES) s << ", stride " << stride.x << "," << stride.y;
        if (dilation != IntPair::ONES) s << ", dilation " << dilation.x << "," << dilation.y;
        if (groups != 1) s << ", " << groups << " groups";
        if (padBefore != IntPair::ZEROS || padAfter != IntPair::ZEROS)
            s << ", padding " << padBefore.x << "," << padBefore.y << ", " << padAfter.x << "," << padAfter.y;
        if (realValuedInput) s << ", real-valued";
        return s.str();
    }

    const Shape& getInputShape() const { return inputShape; }
    const Shape& getFilterShape() const { return filterShape; }
    const IntPair& getStride() const { return stride; }
    const IntPair& getDilation() const { return dilation; }
    int getGroups() const { return groups; }
    Algebra getAlgebra() const { return algebra; }
    DataFormat getDataFormat() const { return dataFormat; }
    FilterLayout getFilterLayout() const { return filterLayout; }
    bool isRealValuedInput() const { return realValuedInput; }
    IntPair getPaddingBefore() const { return padBefore; }
    IntPair getPaddingAfter() const { return padAfter; }
};

class Conv2DFwdDescriptor : public Conv2DDescriptor {
    bool useBias;

public:
    Conv2DFwdDescriptor(const Shape& inputShape, const Shape& filterShape, IntPair stride, IntPair dilation, Padding paddingPreset,
                        const IntTuple& explicitPadding, int groups, Algebra algebra, DataFormat dataFormat,
                        FilterLayout filterLayout, bool useBias, bool realValuedInput = false)
        : Conv2DDescriptor(inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra, dataFormat,
                           filterLayout, realValuedInput), useBias(useBias) {}

    bool operator==(const Conv2DFwdDescriptor& o) const { return key() == o.key() && useBias == o.useBias; }
    bool operator<(const Conv2DFwdDescriptor& o) const { return std::make_tuple(key(), useBias) < std::make_tuple(o.key(), o.useBias); }
    bool isBiasUsed() const { return useBias; }
    Shape getBiasShape() const {
        if (!useBias) return Shape::EMPTY;
        const int channels = Conv2DFilterLayout(filterLayout, algebra).numOutputChannels(filterShape);
        if (algebra == Algebra::REAL) return Shape{channels};
        return Shape{MULTIVECTOR_DIM[algebra], channels};
    }
    std::string toString() const { return Conv2DDescriptor::toString() + (useBias ? ", with bias" : ""); }
};

class Conv2DBwdDescriptor : public Conv2DDescriptor {
    bool requireInputGrad;

public:
    Conv2DBwdDescriptor(const Shape& inputShape, const Shape& filterShape, IntPair stride, IntPair dilation, Padding paddingPreset,
                        const IntTuple& explicitPadding, int groups, Algebra algebra, DataFormat dataFormat,
                        FilterLayout filterLayout, bool requireInputGrad = true, bool realValuedInput = false)
        : Conv2DDescriptor(inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra, dataFormat,
                           filterLayout, realValuedInput), requireInputGrad(requireInputGrad) {}

    bool operator==(const Conv2DBwdDescriptor& o) const { return key() == o.key() && requireInputGrad == o.requireInputGrad; }
    bool operator<(const Conv2DBwdDescriptor& o) const { return std::make_tuple(key(), requireInputGrad) < std::make_tuple(o.key(), o.requireInputGrad); }
    bool isInputGradientRequired() const { return requireInputGrad; }
    std::string toString() const { return Conv2DDescriptor::toString() + (requireInputGrad ? ", with input gradient" : ""); }
};

class DenseDescriptor {
protected:
    Shape inputShape, filterShape;
    Algebra algebra;
    FilterLayout filterLayout;

    auto key() const {
        return std::make_tuple(std::vector<int>(inputShape.getShapePtr(), inputShape.getShapePtr() + inputShape.getSize()),
                               std::vector<int>(filterShape.getShapePtr(), filterShape.getShapePtr() + filterShape.getSize()),
                               (int)algebra, (int)filterLayout);
    }

public:
    DenseDescriptor(const Shape& inputShape, const Shape& filterShape, Algebra algebra, FilterLayout filterLayout)
        : inputShape(inputShape), filterShape(filterShape), algebra(algebra), filterLayout(filterLayout) {}

    int getOutputChannels() const {
        const int idx = algebra == Algebra::REAL ? 0 : 1;   // the outermost filter dimension is the multivector one
        if (filterLayout == FilterLayout::IO) return filterShape[idx + 1];
        if (filterLayout == FilterLayout::OI) return filterShape[idx];
        throw std::runtime_error("Invalid data format");
    }
    int getInputChannels() const {
        const int idx = algebra == Algebra::REAL ? 0 : 1;
        if (filterLayout == FilterLayout::IO) return filterShape[idx];
        if (filterLayout == FilterLayout::OI) return filterShape[idx + 1];
        throw std::runtime_error("Invalid data format");
    }
    Shape getInputShape() const { return inputShape; }
    Shape getFilterShape() const { return filterShape; }
    Shape getOutputShape() const { return Shape{inputShape[0], getOutputChannels()}; }
    Shape getBiasShape() const {
        if (algebra == Algebra::REAL) return Shape{getOutputChannels()};
        return Shape{MULTIVECTOR_DIM[algebra], getOutputChannels()};
    }
    Algebra getAlgebra() const { return algebra; }
    FilterLayout getFilterLayout() const { return filterLayout; }
    std::string toString() const { return ""; }
};

class DenseFwdDescriptor : public DenseDescriptor {
    bool useBias;

public:
    DenseFwdDescriptor(const Shape& inputShape, const Shape& filterShape, Algebra algebra, FilterLayout filterLayout, bool useBias)
        : DenseDescriptor(inputShape, filterShape, algebra, filterLayout), useBias(useBias) {}
    bool operator==(const DenseFwdDescriptor& o) const { return key() == o.key() && useBias == o.useBias; }
    bool operator<(const DenseFwdDescriptor& o) const { return std::make_tuple(key(), useBias) < std::make_tuple(o.key(), o.useBias); }
    bool isBiasUsed() const { return useBias; }
};

class DenseBwdDescriptor : public DenseDescriptor {
    bool requireInputGrad;

public:
    DenseBwdDescriptor(const Shape& inputShape, const Shape& filterShape, Algebra algebra, FilterLayout filterLayout, bool requireInputGrad)
        : DenseDescriptor(inputShape, filterShape, algebra, filterLayout), requireInputGrad(requireInputGrad) {}
    bool operator==(const DenseBwdDescriptor& o) const { return key() == o.key() && requireInputGrad == o.requireInputGrad; }
    bool operator<(const DenseBwdDescriptor& o) const { return std::make_tuple(key(), requireInputGrad) < std::make_tuple(o.key(), o.requireInputGrad); }
    bool isInputGradientRequired() const { return requireInputGrad; }
};

}  // namespace upstride
