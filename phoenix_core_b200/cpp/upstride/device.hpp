// Context (run-time policy), temporary-memory protocol, operation cache and the CUDA device of the
// operator layer. Follows upstride::Context (src/backend/backend.hpp:45-74, src/backend/backend.cc:35-57),
// Allocator / Pointer / MemoryRequest (src/backend/memory_request.hpp:15-114), Operation
// (src/backend/operation.hpp:10-24), OpCollection / GlobalOpCollection (src/backend/op_collections.hpp:121-144,
// src/backend/op_collections.cc:6-64) and device::CUDA (src/backend/cudnn/device.hpp:13-229). There is no
// cuDNN / cuBLAS handle and no helper thread: the device is a CUDA stream, a mutex, a grow-only workspace
// and the caches.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <functional>
#include <list>
#include <map>
#include <memory>
#include <mutex>

#include "descriptors.hpp"

namespace upstride {

enum class ConvFp16ComputePolicy { FULL_16, FORWARD_16_BACKWARD_32, FULL_32 };

class Context {
    bool envOptimizeMemoryUse;
    ConvFp16ComputePolicy convFp16ComputePolicy;
    bool verbose;

    static std::string env(const char* name) { const char* v = std::getenv(name); return v ? std::string(v) : std::string(); }
    static long envInt(const char* name) { const char* v = std::getenv(name); return v ? std::strtol(v, nullptr, 10) : 0; }

public:
    // Reads UPSTRIDE_MEMORY_OPTIMIZED (> 0: 16-product formulation), UPSTRIDE_CONV_FP16_POLICY ("full16",
    // "backward32", anything else: fp32 compute) and UPSTRIDE_VERBOSE once.
    Context() : envOptimizeMemoryUse(envInt("UPSTRIDE_MEMORY_OPTIMIZED") > 0), verbose(envInt("UPSTRIDE_VERBOSE") > 0) {
        const std::string p = env("UPSTRIDE_CONV_FP16_POLICY");
        convFp16ComputePolicy = p == "full16" ? ConvFp16ComputePolicy::FULL_16
                              : p == "backward32" ? ConvFp16ComputePolicy::FORWARD_16_BACKWARD_32 : ConvFp16ComputePolicy::FULL_32;
    }
    virtual ~Context() {}
    bool preferSpeedToMemory() const { return !envOptimizeMemoryUse; }
    bool isFp16ConvForwardAllowed() const {
        return convFp16ComputePolicy == ConvFp16ComputePolicy::FULL_16 || convFp16ComputePolicy == ConvFp16ComputePolicy::FORWARD_16_BACKWARD_32;
    }
    bool isFp16ConvBackwardAllowed() const { return convFp16ComputePolicy == ConvFp16ComputePolicy::FULL_16; }
    ConvFp16ComputePolicy getConvFp16ComputePolicy() const { return convFp16ComputePolicy; }
    bool isVerbose() const { return verbose; }
    virtual void cleanUp() {}
};

class Allocator {
public:
    virtual ~Allocator() {}
    virtual void* mallocTemp(size_t size) = 0;
    virtual size_t getAlignmentConstraint() const = 0;
};

// Base of every cached operation; remembers the largest temporary-memory request it has made.
class Operation {
    size_t memoryNeeds = 0;

public:
    virtual ~Operation() {}
    void updateMemoryNeeds(size_t bytes) { memoryNeeds = std::max(memoryNeeds, bytes); }
    size_t getMemoryNeeds() const { return memoryNeeds; }
};

class MemoryRequest;

// Offset into a memory request; resolves to an address once the request has been submitted.
class Pointer {
    friend class MemoryRequest;
    MemoryRequest* request;
    size_t shift;
    Pointer(MemoryRequest& request, size_t shift) : request(&request), shift(shift) {}

public:
    Pointer() : request(nullptr), shift(0) {}
    void* data();
    operator void*() { return data(); }
    template <typename T> T* cast() { return static_cast<T*>(data()); }
    Pointer operator+(size_t s) const { return Pointer(*request, shift + s); }
};

// Two-phase temporary allocation: alloc() hands out aligned offsets, submit() asks the allocator for one
// block covering them all, Pointer::data() is valid afterwards and until the operation returns.
class MemoryRequest {
    friend class Pointer;
    Allocator& allocator;
    Operation& operation;
    uint8_t* address = nullptr;
    size_t size = 0;
    bool submitted = false;

public:
    MemoryRequest(Allocator& allocator, Operation& operation) : allocator(allocator), operation(operation) {}
    ~MemoryRequest() { operation.updateMemoryNeeds(size); }
    Pointer alloc(size_t bytes) {
        if (submitted) throw std::runtime_error("Memory request is already submitted");
        const size_t align = std::max<size_t>(allocator.getAlignmentConstraint(), 1);
        size = (size + align - 1) / align * align;
        Pointer p(*this, size);
        size += bytes;
        return p;
    }
    void submit() {
        if (size > 0) address = static_cast<uint8_t*>(allocator.mallocTemp(size));
        submitted = true;
    }
    bool isValid() const { return address != nullptr || size == 0; }
    size_t getSize() const { return size; }
};

inline void* Pointer::data() {
    if (!request || !request->submitted) throw std::runtime_error("Accessing a pointer of a memory request that is not submitted");
    return request->address + shift;
}

// Descriptor -> operation cache with a most-recently-used list shared by all operation kinds of a
// device; when more than 200 operations exist the 100 most recently used are kept.
class GlobalOpCollection {
    std::list<Operation*> mru;

public:
    static const size_t GC_THRESHOLD = 200, GC_KEEP = 100;
    void touch(Operation* op) { mru.remove(op); mru.push_front(op); }
    void forget(Operation* op) { mru.remove(op); }
    size_t size() const { return mru.size(); }
    // Returns the operations to drop (least recently used first) once the threshold is exceeded.
    std::vector<Operation*> collect() {
        std::vector<Operation*> drop;
        if (mru.size() <= GC_THRESHOLD) return drop;
        while (mru.size() > GC_KEEP) { drop.push_back(mru.back()); mru.pop_back(); }
        return drop;
    }
};

template <class Descriptor>
class OpCollection {
    GlobalOpCollection& all;
    std::map<Descriptor, std::unique_ptr<Operation>> ops;

public:
    explicit OpCollection(GlobalOpCollection& all) : all(all) {}
    void drop(const std::vector<Operation*>& victims) {
        for (auto it = ops.begin(); it != ops.end();) {
            if (std::find(victims.begin(), victims.end(), it->second.get()) != victims.end()) it = ops.erase(it);
            else ++it;
        }
    }
    template <class DeviceClass, class OperationClass>
    OperationClass& get(DeviceClass& device, const Descriptor& descriptor, const std::function<void(const std::vector<Operation*>&)>& gc) {
        auto it = ops.find(descriptor);
        if (it == ops.end()) {
            gc(all.collect());
            it = ops.emplace(descriptor, std::unique_ptr<Operation>(new OperationClass(device, descriptor))).first;
        }
        all.touch(it->second.get());
        return static_cast<OperationClass&>(*it->second);
    }
    size_t size() const { return ops.size(); }
};

class Device : public Allocator {
    Context& context;
    GlobalOpCollection allOps;
    OpCollection<Conv2DFwdDescriptor> conv2dFwdOps;
    OpCollection<Conv2DBwdDescriptor> conv2dBwdOps;
    OpCollection<DenseFwdDescriptor> denseFwdOps;
    OpCollection<DenseBwdDescriptor> denseBwdOps;
    std::mutex accessControl;
    void* workspace = nullptr;
    size_t workspaceSize = 0;

    void gc(const std::vector<Operation*>& victims) {
        if (victims.empty()) return;
        conv2dFwdOps.drop(victims); conv2dBwdOps.drop(victims); denseFwdOps.drop(victims); denseBwdOps.drop(victims);
    }

protected:
    virtual void* malloc(size_t size) = 0;
    virtual void free(void* memory) = 0;

public:
    explicit Device(Context& context)
        : context(context), conv2dFwdOps(allOps), conv2dBwdOps(allOps), denseFwdOps(allOps), denseBwdOps(allOps) {}
    Device(const Device&) = delete;
    virtual ~Device() {}

    Context& getContext() { return context; }
    std::mutex& getAccessControl() { return accessControl; }

    template <class DeviceClass, class OperationClass>
    OperationClass& getConv2DFwdOperation(const Conv2DFwdDescriptor& d) {
        return conv2dFwdOps.get<DeviceClass, OperationClass>(static_cast<DeviceClass&>(*this), d, [this](const std::vector<Operation*>& v) { gc(v); });
    }
    template <class DeviceClass, class OperationClass>
    OperationClass& getConv2DBwdOperation(const Conv2DBwdDescriptor& d) {
        return conv2dBwdOps.get<DeviceClass, OperationClass>(static_cast<DeviceClass&>(*this), d, [this](const std::vector<Operation*>& v) { gc(v); });
    }
    template <class DeviceClass, class OperationClass>
    OperationClass& getDenseFwdOperation(const DenseFwdDescriptor& d) {
        return denseFwdOps.get<DeviceClass, OperationClass>(static_cast<DeviceClass&>(*this), d, [this](const std::vector<Operation*>& v) { gc(v); });
    }
    template <class DeviceClass, class OperationClass>
    OperationClass& getDenseBwdOperation(const DenseBwdDescriptor& d) {
        return denseBwdOps.get<DeviceClass, OperationClass>(static_cast<DeviceClass&>(*this), d, [this](const std::vector<Operation*>& v) { gc(v); });
    }
    size_t getNumCachedOperations() const { return allOps.size(); }

    // One workspace per device that only grows; operations carve their temporaries out of it.
    void* requestWorkspaceMemory(size_t size) {
        if (size > workspaceSize) {
            free(workspace);
            workspace = malloc(size);
            workspaceSize = size;
        }
        return workspace;
    }
    void freeWorkspaceMemory() { free(workspace); workspace = nullptr; workspaceSize = 0; }
    size_t getWorkspaceSize() const { return workspaceSize; }
    void* mallocTemp(size_t size) override { return requestWorkspaceMemory(size); }
    size_t getAlignmentConstraint() const override { return 1; }
};

namespace device {

// One CUDA device as seen through one stream: every operation is enqueued on that stream and nothing
// synchronises it except explicit host copies.
class CUDA : public Device {
    cudaStream_t cudaStream;

protected:
    void* malloc(size_t size) override {
        void* p = nullptr;
        if (size == 0) return nullptr;
        if (cudaMalloc(&p, size) != cudaSuccess) throw std::runtime_error("CUDA memory allocation failed");
        return p;
    }
    void free(void* memory) override {
        if (memory) { cudaStreamSynchronize(cudaStream); cudaFree(memory); }
    }

public:
    explicit CUDA(Context& context, cudaStream_t stream = nullptr) : Device(context), cudaStream(stream) {}
    ~CUDA() override { freeWorkspaceMemory(); }
    cudaStream_t stream() const { return cudaStream; }
    size_t getAlignmentConstraint() const override { return 256; }
    void zero(void* ptr, size_t bytes) {
        if (cudaMemsetAsync(ptr, 0, bytes, cudaStream) != cudaSuccess) throw std::runtime_error("cudaMemsetAsync failed");
    }
    void synchronize() { if (cudaStreamSynchronize(cudaStream) != cudaSuccess) throw std::runtime_error("stream synchronisation failed"); }
    // Reads back the wait status the kernels of the last operation left in the workspace (synchronises the stream) and
    // throws std::runtime_error if a bounded device-side wait expired. The reference checks a library status after every
    // cuDNN / cuBLAS call (src/backend/cudnn/context.hpp:68-110); the fused kernels report through this word instead.
    void checkDeviceStatus();
};

}  // namespace device

namespace cuda {

// The devices of a process, one per CUDA stream, created on first use and kept until cleanUp()
// (reference: cudnn::Context::registerDevice / cleanUp, src/backend/cudnn/cudnn.cc:5-22, context.hpp:51-56).
// A framework plugin calls registerDevice(stream) with the stream of the current operator invocation and runs
// the operation on the device it gets; two streams never share a workspace or an operation cache.
class Context : public upstride::Context {
    std::map<cudaStream_t, std::unique_ptr<device::CUDA>> devices;
    std::mutex mutex;

public:
    device::CUDA& registerDevice(const cudaStream_t& stream) {
        std::lock_guard<std::mutex> lock(mutex);
        auto entry = devices.find(stream);
        if (entry == devices.end()) entry = devices.emplace(stream, std::unique_ptr<device::CUDA>(new device::CUDA(*this, stream))).first;
        return *entry->second;
    }
    size_t getNumDevices() {
        std::lock_guard<std::mutex> lock(mutex);
        return devices.size();
    }
    void cleanUp() override {
        std::lock_guard<std::mutex> lock(mutex);
        devices.clear();
    }
};

}  // namespace cuda
}  // namespace upstride
