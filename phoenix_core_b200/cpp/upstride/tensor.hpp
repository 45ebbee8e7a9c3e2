// Tensors of the operator layer: a non-owning view (pointer + shape + device), views of the equal blocks
// along the outermost axis (this is the "four quaternion components stacked on the batch axis" layout),
// and an owning tensor for tests and tools. Follows upstride::Tensor / TensorSplit / AllocatedTensor
// (src/backend/tensor.hpp:386-581, src/backend/cudnn/tensor.hpp:15-67).
#pragma once

#include <cuda_runtime.h>

#include <vector>

#include "types.hpp"

namespace upstride {

inline void cudaCheck(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename Device, typename T>
class Tensor {
    Device& device;
    Shape shape;
    T* ptr;

public:
    Tensor(Device& device, const Shape& shape, T* ptr) : device(device), shape(shape), ptr(ptr) {}
    // const view of a mutable tensor
    template <typename U, typename = typename std::enable_if<std::is_same<const U, T>::value>::type>
    Tensor(const Tensor<Device, U>& other) : device(other.getDevice()), shape(other.getShape()), ptr(other.getDataPtr()) {}

    T* getDataPtr() const { return ptr; }
    const Shape& getShape() const { return shape; }
    Device& getDevice() const { return device; }
    Tensor<Device, T> slice(int index, const Shape& partShape) const { return Tensor<Device, T>(device, partShape, ptr + (size_t)index * partShape.numel()); }
    // Sets every element to zero, in stream order.
    void zero() { device.zero(ptr, (size_t)shape.numel() * sizeof(T)); }
};

// PARTS equal blocks along the outermost dimension. keepOutermostDimension == false drops the leading
// axis from the part shape (used for filters [4, Co, Ci, kh, kw] -> [Co, Ci, kh, kw]).
template <typename Device, typename T, int PARTS>
class TensorSplit {
    std::vector<Tensor<Device, T>> parts;
    Shape partShape;

public:
    TensorSplit(const Tensor<Device, T>& tensor, bool keepOutermostDimension = true)
        : partShape(keepOutermostDimension ? tensor.getShape().split(PARTS) : tensor.getShape().slice(1)) {
        if (!keepOutermostDimension && tensor.getShape()[0] != PARTS) throw std::invalid_argument("Outermost dimension mismatch in a tensor split");
        for (int i = 0; i < PARTS; ++i) parts.push_back(tensor.slice(i, partShape));
    }
    Tensor<Device, T>& operator[](int i) { return parts[(size_t)i]; }
    const Tensor<Device, T>& operator[](int i) const { return parts[(size_t)i]; }
    const Shape& shape() const { return partShape; }
};

// Owns device memory. Assignment from / conversion to std::vector copy through the device's stream and
// synchronise it, which is what tests need.
template <typename Device, typename T>
class AllocatedTensor : public Tensor<Device, T> {
    static T* allocate(const Shape& shape) {
        void* p = nullptr;
        const size_t bytes = (size_t)std::max(shape.numel(), 1) * sizeof(T);
        cudaCheck(cudaMalloc(&p, bytes), "cudaMalloc");
        return static_cast<T*>(p);
    }

public:
    AllocatedTensor(Device& device, const Shape& shape) : Tensor<Device, T>(device, shape, allocate(shape)) {}
    AllocatedTensor(const AllocatedTensor&) = delete;
    ~AllocatedTensor() { cudaFree(this->getDataPtr()); }

    AllocatedTensor& operator=(const std::vector<T>& host) {
        if ((int)host.size() != this->getShape().numel()) throw std::invalid_argument("Cannot copy tensor content from a vector of a different size");
        cudaCheck(cudaMemcpyAsync(this->getDataPtr(), host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice, this->getDevice().stream()), "cudaMemcpyAsync");
        cudaCheck(cudaStreamSynchronize(this->getDevice().stream()), "cudaStreamSynchronize");
        return *this;
    }
    operator std::vector<T>() const {
        std::vector<T> host((size_t)this->getShape().numel());
        cudaCheck(cudaMemcpyAsync(host.data(), this->getDataPtr(), host.size() * sizeof(T), cudaMemcpyDeviceToHost, this->getDevice().stream()), "cudaMemcpyAsync");
        cudaCheck(cudaStreamSynchronize(this->getDevice().stream()), "cudaStreamSynchronize");
        return host;
    }
};

}  // namespace upstride
