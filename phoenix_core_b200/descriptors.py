"""Operation descriptors with the reference's names, argument order and error behaviour.

Mirrors ``upstride::Conv2DDescriptor`` / ``Conv2DFwdDescriptor`` / ``Conv2DBwdDescriptor``
(reference ``src/backend/conv2d_descriptor.hpp:113-423``), ``DenseFwdDescriptor`` / ``DenseBwdDescriptor``
(``src/backend/dense_descriptor.hpp:11-131``), the enums of ``src/backend/types.hpp:76-97`` and ``src/algebras.hpp:17-27``,
and the TF-style geometry rule of ``src/utils.cc:10-50``.
"""
import enum


class Algebra(enum.IntEnum):
    REAL = 0
    COMPLEX = 1
    QUATERNION = 2
    GA_300 = 3


MULTIVECTOR_DIM = {Algebra.REAL: 1, Algebra.COMPLEX: 2, Algebra.QUATERNION: 4, Algebra.GA_300: 8}


class Padding(enum.IntEnum):
    SAME = 0
    VALID = 1
    EXPLICIT = 2


class DataFormat(enum.IntEnum):
    NCHW = 0   # channel-first
    NHWC = 1   # channel-last
    NC = 2


class FilterLayout(enum.IntEnum):
    OIHW = 0
    OHWI = 1
    HWIO = 2
    IO = 3
    OI = 4


def padding_from_string(text):
    try:
        return Padding[text.upper()]
    except KeyError:
        raise ValueError("Invalid padding encountered: " + text)


def data_format_from_string(text):
    try:
        return DataFormat[text.upper()]
    except KeyError:
        raise ValueError("Invalid data format encountered: " + text)


def filter_layout_from_string(text):
    try:
        return FilterLayout[text.upper()]
    except KeyError:
        raise ValueError("Invalid filter layout encountered: " + text)


def compute_windowed_output_size_and_padding(input_size, filter_size, dilation, stride, padding=None,
                                             padding_before=None, padding_after=None):
    """Two call forms, as the reference's overloads (``src/utils.cc:10-50``):

    * with a ``Padding`` preset (SAME / VALID): returns ``(output size, padding before, padding after)``;
    * with explicit ``padding_before`` / ``padding_after``: returns the output size.
    """
    effective = (filter_size - 1) * dilation + 1
    if padding is None or padding == Padding.EXPLICIT:
        return (input_size + padding_before + padding_after - effective + stride) // stride
    if padding == Padding.VALID:
        return (input_size - effective + stride) // stride, 0, 0
    if padding == Padding.SAME:
        out = (input_size + stride - 1) // stride
        needed = max(0, (out - 1) * stride + effective - input_size)
        # for odd totals the extra pixel goes after (bottom / right)
        return out, needed // 2, needed - needed // 2
    raise ValueError("Invalid padding")


def _pair(v):
    if isinstance(v, int):
        return (v, v)
    v = tuple(v)
    if len(v) == 1:
        return (v[0], v[0])
    if len(v) == 2:
        return v
    raise ValueError("expected one or two integers, got %r" % (v,))


def _dims(data_format):
    """Indices of (channel, height, width) in a 4-D activation shape."""
    if data_format == DataFormat.NCHW:
        return 1, 2, 3
    if data_format == DataFormat.NHWC:
        return 3, 1, 2
    raise ValueError("Invalid data format for a convolution")


def _filter_dims(layout, algebra):
    """Indices of (out channels, in channels, height, width) in the filter shape."""
    off = 0 if algebra == Algebra.REAL else 1
    if layout == FilterLayout.OIHW:
        o, i, h, w = 0, 1, 2, 3
    elif layout == FilterLayout.OHWI:
        o, h, w, i = 0, 1, 2, 3
    elif layout == FilterLayout.HWIO:
        h, w, i, o = 0, 1, 2, 3
    else:
        raise ValueError("Invalid filter layout for a convolution")
    return o + off, i + off, h + off, w + off


class Conv2DDescriptor:
    def __init__(self, inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra,
                 dataFormat, filterLayout, realValuedInput=False):
        self.inputShape = tuple(inputShape)
        self.filterShape = tuple(filterShape)
        self.stride = _pair(stride)
        self.dilation = _pair(dilation)
        self.groups = groups
        self.algebra = Algebra(algebra)
        self.dataFormat = DataFormat(dataFormat)
        self.filterLayout = FilterLayout(filterLayout)
        self.realValuedInput = bool(realValuedInput)

        if len(self.inputShape) != 4:
            raise ValueError("Four-dimensional input tensor expected")
        if self.algebra != Algebra.REAL:
            if len(self.filterShape) != 5:
                raise ValueError("Five-dimensional filter tensor expected")
            if self.filterShape[0] != MULTIVECTOR_DIM[self.algebra]:
                raise ValueError("First filter dimension mismatch, got %d" % self.filterShape[0])
        elif len(self.filterShape) != 4:
            raise ValueError("Four-dimensional filter tensor expected")

        _, hd, wd = _dims(self.dataFormat)
        _, _, fh, fw = _filter_dims(self.filterLayout, self.algebra)
        paddingPreset = Padding(paddingPreset)
        if paddingPreset == Padding.EXPLICIT:
            ep = tuple(explicitPadding)
            self.padBefore = (ep[0], ep[1])
            self.padAfter = (ep[2], ep[3])
        else:
            _, bh, ah = compute_windowed_output_size_and_padding(self.inputShape[hd], self.filterShape[fh],
                                                                 self.dilation[0], self.stride[0], paddingPreset)
            _, bw, aw = compute_windowed_output_size_and_padding(self.inputShape[wd], self.filterShape[fw],
                                                                 self.dilation[1], self.stride[1], paddingPreset)
            self.padBefore = (bh, bw)
            self.padAfter = (ah, aw)

    # accessors with the reference's names
    def getInputShape(self): return self.inputShape
    def getFilterShape(self): return self.filterShape
    def getStride(self): return self.stride
    def getDilation(self): return self.dilation
    def getGroups(self): return self.groups
    def getAlgebra(self): return self.algebra
    def getDataFormat(self): return self.dataFormat
    def getFilterLayout(self): return self.filterLayout
    def isRealValuedInput(self): return self.realValuedInput
    def getPaddingBefore(self): return self.padBefore
    def getPaddingAfter(self): return self.padAfter

    def numOutputChannels(self):
        o, _, _, _ = _filter_dims(self.filterLayout, self.algebra)
        return self.filterShape[o]

    def getOutputShape(self):
        cd, hd, wd = _dims(self.dataFormat)
        _, _, fh, fw = _filter_dims(self.filterLayout, self.algebra)
        out = [0, 0, 0, 0]
        out[0] = self.inputShape[0]
        out[cd] = self.numOutputChannels()
        out[hd] = compute_windowed_output_size_and_padding(self.inputShape[hd], self.filterShape[fh], self.dilation[0],
                                                           self.stride[0], None, self.padBefore[0], self.padAfter[0])
        out[wd] = compute_windowed_output_size_and_padding(self.inputShape[wd], self.filterShape[fw], self.dilation[1],
                                                           self.stride[1], None, self.padBefore[1], self.padAfter[1])
        if self.realValuedInput:
            out[0] *= MULTIVECTOR_DIM[self.algebra]
        return tuple(out)

    def _key(self):
        return (self.inputShape, self.filterShape, self.stride, self.dilation, self.groups, int(self.algebra),
                int(self.dataFormat), self.realValuedInput, self.padBefore, self.padAfter)

    def __eq__(self, other):
        return type(self) is type(other) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())


class Conv2DFwdDescriptor(Conv2DDescriptor):
    def __init__(self, inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra,
                 dataFormat, filterLayout, useBias, realValuedInput=False):
        super().__init__(inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra,
                         dataFormat, filterLayout, realValuedInput)
        self.useBias = bool(useBias)

    def isBiasUsed(self): return self.useBias

    def getBiasShape(self):
        if not self.useBias:
            return ()
        channels = self.numOutputChannels()
        if self.algebra == Algebra.REAL:
            return (channels,)
        return (MULTIVECTOR_DIM[self.algebra], channels)

    def _key(self):
        return super()._key() + (self.useBias,)


class Conv2DBwdDescriptor(Conv2DDescriptor):
    def __init__(self, inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra,
                 dataFormat, filterLayout, requireInputGrad=True, realValuedInput=False):
        super().__init__(inputShape, filterShape, stride, dilation, paddingPreset, explicitPadding, groups, algebra,
                         dataFormat, filterLayout, realValuedInput)
        self.requireInputGrad = bool(requireInputGrad)

    def isInputGradientRequired(self): return self.requireInputGrad

    def _key(self):
        return super()._key() + (self.requireInputGrad,)


class DenseDescriptor:
    def __init__(self, inputShape, filterShape, algebra, filterLayout):
        self.inputShape = tuple(inputShape)
        self.filterShape = tuple(filterShape)
        self.algebra = Algebra(algebra)
        self.filterLayout = FilterLayout(filterLayout)

    def getOutputChannels(self):
        idx = 0 if self.algebra == Algebra.REAL else 1
        if self.filterLayout == FilterLayout.IO:
            return self.filterShape[idx + 1]
        if self.filterLayout == FilterLayout.OI:
            return self.filterShape[idx]
        raise RuntimeError("Invalid data format")

    def getInputChannels(self):
        idx = 0 if self.algebra == Algebra.REAL else 1
        return self.filterShape[idx] if self.filterLayout == FilterLayout.IO else self.filterShape[idx + 1]

    def getInputShape(self): return self.inputShape
    def getFilterShape(self): return self.filterShape
    def getOutputShape(self): return (self.inputShape[0], self.getOutputChannels())
    def getAlgebra(self): return self.algebra
    def getFilterLayout(self): return self.filterLayout

    def getBiasShape(self):
        if self.algebra == Algebra.REAL:
            return (self.getOutputChannels(),)
        return (MULTIVECTOR_DIM[self.algebra], self.getOutputChannels())


class DenseFwdDescriptor(DenseDescriptor):
    def __init__(self, inputShape, filterShape, algebra, filterLayout, useBias):
        super().__init__(inputShape, filterShape, algebra, filterLayout)
        self.useBias = bool(useBias)

    def isBiasUsed(self): return self.useBias


class DenseBwdDescriptor(DenseDescriptor):
    def __init__(self, inputShape, filterShape, algebra, filterLayout, requireInputGrad):
        super().__init__(inputShape, filterShape, algebra, filterLayout)
        self.requireInputGrad = bool(requireInputGrad)

    def isInputGradientRequired(self): return self.requireInputGrad
