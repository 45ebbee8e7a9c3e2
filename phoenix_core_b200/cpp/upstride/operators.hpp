// Operator classes of the layer: UpstrideConv2DFunctor, UpstrideConv2DGradFunctor, UpstrideDenseFunctor,
// UpstrideDenseGradFunctor with the algebra-select mixin (reference: src/conv2d.hpp:23-564,
// src/dense.hpp:21-379, src/algebra_select_mixin.hpp:21-50). For device::CUDA the quaternion branch hands the
// whole operation to the fused kernels behind the C ABI -- the slot the reference gives its custom 1x1
// kernels (src/conv2d.hpp:117, :380), widened to every quaternion convolution and to dense. The formulation
// (8-product by default, 16-product when memory-optimised) and the fp16 policy still come from the Context.
// Every algebra of the enum goes through the same kernels with its own signed block.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <functional>

#include "../../../include/phoenix_core_b200.h"
#include "device.hpp"
#include "tensor.hpp"

namespace upstride {

// Runtime algebra -> compile-time template argument.
template <class OperationClass>
class AlgebraSelectionMixin {
protected:
    template <typename... Args>
    void proceedWithAlgebra(Algebra algebra, Args&&... args) {
        OperationClass& self = static_cast<OperationClass&>(*this);
        switch (algebra) {
            case Algebra::REAL: self.template proceedWithAlgebra<Algebra::REAL>(std::forward<Args>(args)...); return;
            case Algebra::COMPLEX: self.template proceedWithAlgebra<Algebra::COMPLEX>(std::forward<Args>(args)...); return;
            case Algebra::QUATERNION: self.template proceedWithAlgebra<Algebra::QUATERNION>(std::forward<Args>(args)...); return;
            case Algebra::GA_300: self.template proceedWithAlgebra<Algebra::GA_300>(std::forward<Args>(args)...); return;
        }
        throw std::invalid_argument("Invalid algebra");
    }
};

template <typename T> struct DataTypeCode;
template <> struct DataTypeCode<float> { static const int value = PCB_F32; };
template <> struct DataTypeCode<__half> { static const int value = PCB_F16; };
template <> struct DataTypeCode<__nv_bfloat16> { static const int value = PCB_BF16; };

// Maps a status of the C ABI to the exception classes of the reference.
inline void checkStatus(int status) {
    if (status == PCB_OK) return;
    const std::string msg = std::string("phoenix_core_b200: ") + pcb_last_error_message();
    if (status == PCB_ERR_INVALID_ARGUMENT) throw std::invalid_argument(msg);
    throw std::runtime_error(msg + " (" + pcb_status_string(status) + ")");
}

inline void device::CUDA::checkDeviceStatus() {
    if (getWorkspaceSize() > 0) checkStatus(pcb_check_device_status(requestWorkspaceMemory(0), getWorkspaceSize(), cudaStream));
}

inline int fp16PolicyCode(const Context& c) {
    switch (c.getConvFp16ComputePolicy()) {
        case ConvFp16ComputePolicy::FULL_16: return PCB_FP16_POLICY_FULL16;
        case ConvFp16ComputePolicy::FORWARD_16_BACKWARD_32: return PCB_FP16_POLICY_BACKWARD32;
        default: return PCB_FP16_POLICY_FULL32;
    }
}

// upstride::Algebra -> pcb_algebra (the C ABI keeps the quaternion algebra at zero).
inline int algebraCode(Algebra a) {
    switch (a) {
        case Algebra::REAL: return PCB_ALGEBRA_REAL;
        case Algebra::COMPLEX: return PCB_ALGEBRA_COMPLEX;
        case Algebra::QUATERNION: return PCB_ALGEBRA_QUATERNION;
        case Algebra::GA_300: return PCB_ALGEBRA_GA_300;
    }
    throw std::invalid_argument("Invalid algebra");
}

inline pcb_conv2d_desc makeConvDesc(const Conv2DDescriptor& d, int dtype, Context& context) {
    const Shape& in = d.getInputShape();
    const Shape& f = d.getFilterShape();
    const int dim = MULTIVECTOR_DIM[d.getAlgebra()];
    const int o = d.getAlgebra() == Algebra::REAL ? 0 : 1;   // real filters carry no leading component axis
    const bool realInput = d.isRealValuedInput() && d.getAlgebra() != Algebra::REAL;
    pcb_conv2d_desc c = {};
    int cd, hd, wd, fo, fi, fh, fw;                          // positions of channels / height / width in the shapes
    switch (d.getDataFormat()) {
        case DataFormat::NCHW: c.data_format = PCB_LAYOUT_NCHW; cd = 1; hd = 2; wd = 3; break;
        case DataFormat::NHWC: c.data_format = PCB_LAYOUT_NHWC; cd = 3; hd = 1; wd = 2; break;
        default: throw std::runtime_error("phoenix_core_b200: unsupported data format for a convolution");
    }
    switch (d.getFilterLayout()) {
        case FilterLayout::OIHW: c.filter_layout = PCB_FILTER_OIHW; fo = o; fi = o + 1; fh = o + 2; fw = o + 3; break;
        case FilterLayout::OHWI: c.filter_layout = PCB_FILTER_OHWI; fo = o; fh = o + 1; fw = o + 2; fi = o + 3; break;
        case FilterLayout::HWIO: c.filter_layout = PCB_FILTER_HWIO; fh = o; fw = o + 1; fi = o + 2; fo = o + 3; break;
        default: throw std::runtime_error("phoenix_core_b200: unsupported filter layout for a convolution");
    }
    if (!realInput && in[0] % dim != 0) throw std::invalid_argument("Outermost input dimension must be a multiple of the multivector dimension");
    if (in[cd] != f[fi] * d.getGroups()) throw std::invalid_argument("Input channels mismatch");
    c.dtype = dtype;
    c.algebra = algebraCode(d.getAlgebra());
    c.n = realInput ? in[0] : in[0] / dim;
    c.ci = f[fi]; c.co = f[fo]; c.h = in[hd]; c.w = in[wd]; c.kh = f[fh]; c.kw = f[fw];
    c.stride_h = d.getStride().x; c.stride_w = d.getStride().y;
    c.dilation_h = d.getDilation().x; c.dilation_w = d.getDilation().y;
    c.pad_top = d.getPaddingBefore().x; c.pad_left = d.getPaddingBefore().y;
    c.pad_bottom = d.getPaddingAfter().x; c.pad_right = d.getPaddingAfter().y;
    c.groups = d.getGroups();
    c.real_valued_input = realInput;
    c.variant = context.preferSpeedToMemory() ? PCB_VARIANT_8_PRODUCT : PCB_VARIANT_16_PRODUCT;
    c.fp16_policy = fp16PolicyCode(context);
    c.engine = PCB_ENGINE_AUTO;
    return c;
}

inline pcb_dense_desc makeDenseDesc(const DenseDescriptor& d, int dtype, Context& context) {
    const Shape in = d.getInputShape();
    const int dim = MULTIVECTOR_DIM[d.getAlgebra()];
    if (in.getSize() != 2 || in[0] % dim != 0) throw std::invalid_argument("Dense input must be [D*batch, features]");
    if (in[1] != d.getInputChannels()) throw std::invalid_argument("Input features mismatch");
    pcb_dense_desc c = {};
    c.dtype = dtype;
    c.algebra = algebraCode(d.getAlgebra());
    c.batch = in[0] / dim;
    c.in_features = in[1];
    c.out_features = d.getOutputChannels();
    c.filter_oi = d.getFilterLayout() == FilterLayout::OI;
    c.variant = context.preferSpeedToMemory() ? PCB_VARIANT_8_PRODUCT : PCB_VARIANT_16_PRODUCT;
    c.engine = PCB_ENGINE_AUTO;
    return c;
}

template <typename Device, typename T>
class UpstrideConv2DFunctor : public AlgebraSelectionMixin<UpstrideConv2DFunctor<Device, T>>, public Operation {
    friend class AlgebraSelectionMixin<UpstrideConv2DFunctor<Device, T>>;
    using AlgebraSelectionMixin<UpstrideConv2DFunctor<Device, T>>::proceedWithAlgebra;
    Device& device;
    const Conv2DFwdDescriptor descriptor;

public:
    UpstrideConv2DFunctor(Device& device, const Conv2DFwdDescriptor& descriptor) : device(device), descriptor(descriptor) {}

    void operator()(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                    const Tensor<Device, const T>* biasTensor, Tensor<Device, T>& outputTensor, const IntPair&, const IntPair&, int = 1) {
        if (inputTensor.getShape().empty()) return;   // an empty batch is a silent no-op
        proceedWithAlgebra(descriptor.getAlgebra(), allocator, inputTensor, kernelTensor, biasTensor, outputTensor);
    }

    template <Algebra algebra>
    void proceedWithAlgebra(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                            const Tensor<Device, const T>* biasTensor, Tensor<Device, T>& outputTensor) {
        if (descriptor.isRealValuedInput() && biasTensor) throw std::runtime_error("Bias addition is not supported for type0 inputs");
        pcb_conv2d_desc c = makeConvDesc(descriptor, DataTypeCode<T>::value, device.getContext());
        c.has_bias = biasTensor != nullptr;
        MemoryRequest memory(allocator, *this);
        Pointer workspace = memory.alloc(pcb_qconv2d_fwd_workspace_size(&c));
        memory.submit();
        checkStatus(pcb_qconv2d_fwd(&c, inputTensor.getDataPtr(), kernelTensor.getDataPtr(), biasTensor ? biasTensor->getDataPtr() : nullptr,
                                    outputTensor.getDataPtr(), workspace.data(), memory.getSize(), device.stream()));
    }
};

template <typename Device, typename T>
class UpstrideConv2DGradFunctor : public AlgebraSelectionMixin<UpstrideConv2DGradFunctor<Device, T>>, public Operation {
    friend class AlgebraSelectionMixin<UpstrideConv2DGradFunctor<Device, T>>;
    using AlgebraSelectionMixin<UpstrideConv2DGradFunctor<Device, T>>::proceedWithAlgebra;
    Device& device;
    const Conv2DBwdDescriptor descriptor;

public:
    UpstrideConv2DGradFunctor(Device& device, const Conv2DBwdDescriptor& descriptor) : device(device), descriptor(descriptor) {}

    void operator()(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                    const Tensor<Device, const T>& gradTensor, Tensor<Device, T>& kernelGradTensor, Tensor<Device, T>& inputGradTensor,
                    const IntPair&, const IntPair&, int = 1) {
        if (inputTensor.getShape().empty()) { kernelGradTensor.zero(); return; }   // an empty batch zeroes the filter gradient
        proceedWithAlgebra(descriptor.getAlgebra(), allocator, inputTensor, kernelTensor, gradTensor, kernelGradTensor, inputGradTensor);
    }

    template <Algebra algebra>
    void proceedWithAlgebra(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                            const Tensor<Device, const T>& gradTensor, Tensor<Device, T>& kernelGradTensor, Tensor<Device, T>& inputGradTensor) {
        if (descriptor.isRealValuedInput() && descriptor.isInputGradientRequired())
            throw std::logic_error("Input gradient required for type0 input tensor");
        pcb_conv2d_desc c = makeConvDesc(descriptor, DataTypeCode<T>::value, device.getContext());
        c.require_input_grad = descriptor.isInputGradientRequired();
        MemoryRequest memory(allocator, *this);
        Pointer workspace = memory.alloc(pcb_qconv2d_bwd_workspace_size(&c));
        memory.submit();
        checkStatus(pcb_qconv2d_bwd(&c, inputTensor.getDataPtr(), kernelTensor.getDataPtr(), gradTensor.getDataPtr(), kernelGradTensor.getDataPtr(),
                                    c.require_input_grad ? inputGradTensor.getDataPtr() : nullptr, workspace.data(), memory.getSize(), device.stream()));
    }
};

template <typename Device, typename T>
class UpstrideDenseFunctor : public AlgebraSelectionMixin<UpstrideDenseFunctor<Device, T>>, public Operation {
    friend class AlgebraSelectionMixin<UpstrideDenseFunctor<Device, T>>;
    using AlgebraSelectionMixin<UpstrideDenseFunctor<Device, T>>::proceedWithAlgebra;
    Device& device;
    const DenseFwdDescriptor descriptor;

public:
    UpstrideDenseFunctor(Device& device, const DenseFwdDescriptor& descriptor) : device(device), descriptor(descriptor) {}

    void operator()(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                    const Tensor<Device, const T>* biasTensor, Tensor<Device, T>& outputTensor) {
        if (inputTensor.getShape().empty()) return;
        proceedWithAlgebra(descriptor.getAlgebra(), allocator, inputTensor, kernelTensor, biasTensor, outputTensor);
    }

    template <Algebra algebra>
    void proceedWithAlgebra(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                            const Tensor<Device, const T>* biasTensor, Tensor<Device, T>& outputTensor) {
        pcb_dense_desc c = makeDenseDesc(descriptor, DataTypeCode<T>::value, device.getContext());
        c.has_bias = biasTensor != nullptr;
        MemoryRequest memory(allocator, *this);
        Pointer workspace = memory.alloc(pcb_qdense_fwd_workspace_size(&c));
        memory.submit();
        checkStatus(pcb_qdense_fwd(&c, inputTensor.getDataPtr(), kernelTensor.getDataPtr(), biasTensor ? biasTensor->getDataPtr() : nullptr,
                                   outputTensor.getDataPtr(), workspace.data(), memory.getSize(), device.stream()));
    }
};

template <typename Device, typename T>
class UpstrideDenseGradFunctor : public AlgebraSelectionMixin<UpstrideDenseGradFunctor<Device, T>>, public Operation {
    friend class AlgebraSelectionMixin<UpstrideDenseGradFunctor<Device, T>>;
    using AlgebraSelectionMixin<UpstrideDenseGradFunctor<Device, T>>::proceedWithAlgebra;
    Device& device;
    const DenseBwdDescriptor descriptor;

public:
    UpstrideDenseGradFunctor(Device& device, const DenseBwdDescriptor& descriptor) : device(device), descriptor(descriptor) {}

    void operator()(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                    const Tensor<Device, const T>& gradTensor, Tensor<Device, T>& kernelGradTensor, Tensor<Device, T>& inputGradTensor) {
        if (inputTensor.getShape().empty()) { kernelGradTensor.zero(); return; }
        proceedWithAlgebra(descriptor.getAlgebra(), allocator, inputTensor, kernelTensor, gradTensor, kernelGradTensor, inputGradTensor);
    }

    template <Algebra algebra>
    void proceedWithAlgebra(Allocator& allocator, const Tensor<Device, const T>& inputTensor, const Tensor<Device, const T>& kernelTensor,
                            const Tensor<Device, const T>& gradTensor, Tensor<Device, T>& kernelGradTensor, Tensor<Device, T>& inputGradTensor) {
        pcb_dense_desc c = makeDenseDesc(descriptor, DataTypeCode<T>::value, device.getContext());
        c.require_input_grad = descriptor.isInputGradientRequired();
        MemoryRequest memory(allocator, *this);
        Pointer workspace = memory.alloc(pcb_qdense_bwd_workspace_size(&c));
        memory.submit();
        checkStatus(pcb_qdense_bwd(&c, inputTensor.getDataPtr(), kernelTensor.getDataPtr(), gradTensor.getDataPtr(), kernelGradTensor.getDataPtr(),
                                   c.require_input_grad ? inputGradTensor.getDataPtr() : nullptr, workspace.data(), memory.getSize(), device.stream()));
    }
};

}  // namespace upstride
