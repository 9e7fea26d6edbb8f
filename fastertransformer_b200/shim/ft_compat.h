// Stand-ins for the few FasterTransformer utility types the decode layers use in their interface
// (Tensor, TensorMap, IAllocator, DataType, MemoryType).  They exist so that the shim classes can be
// built and tested outside a FasterTransformer checkout.  Inside one, define FTB200_WITH_FT_HEADERS and
// the shim includes the project's own headers (utils/Tensor.h, utils/allocator.h) instead; the member
// functions used by the shim have the same names and meaning there.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace fastertransformer {

enum DataType { TYPE_INVALID, TYPE_BOOL, TYPE_UINT8, TYPE_UINT16, TYPE_UINT32, TYPE_UINT64, TYPE_INT8, TYPE_INT16,
                TYPE_INT32, TYPE_INT64, TYPE_FP16, TYPE_FP32, TYPE_FP64, TYPE_BYTES, TYPE_BF16 };
enum MemoryType { MEMORY_CPU, MEMORY_CPU_PINNED, MEMORY_GPU };

struct Tensor {
    MemoryType          where = MEMORY_CPU;
    DataType            type  = TYPE_INVALID;
    std::vector<size_t> shape;
    const void*         data = nullptr;

    Tensor() = default;
    Tensor(MemoryType w, DataType t, std::vector<size_t> s, const void* d): where(w), type(t), shape(std::move(s)), data(d) {}

    size_t size() const
    {
        if (data == nullptr || shape.empty()) {
            return 0;
        }
        size_t n = 1;
        for (size_t d : shape) {
            n *= d;
        }
        return n;
    }
    template<typename T>
    T* getPtr() const
    {
        return (T*)data;
    }
    template<typename T>
    T* getPtrWithOffset(size_t offset) const
    {
        return data == nullptr ? nullptr : ((T*)data) + offset;
    }
    template<typename T>
    T getVal(size_t index = 0) const
    {
        if (where == MEMORY_GPU) {
            throw std::runtime_error("[FT][ERROR] getVal() needs a host tensor");
        }
        return ((const T*)data)[index];
    }
};

class TensorMap {
    std::unordered_map<std::string, Tensor> tensor_map_;

public:
    TensorMap() = default;
    TensorMap(const std::unordered_map<std::string, Tensor>& m)
    {
        for (const auto& kv : m) {
            if (kv.second.size() > 0) {
                tensor_map_.insert(kv);
            }
        }
    }
    bool isExist(const std::string& key) const
    {
        return tensor_map_.find(key) != tensor_map_.end();
    }
    void insert(const std::string& key, const Tensor& value)
    {
        if (isExist(key)) {
            throw std::runtime_error("[FT][ERROR] Duplicated key " + key);
        }
        if (value.size() > 0) {
            tensor_map_.insert({key, value});
        }
    }
    Tensor& at(const std::string& key)
    {
        auto it = tensor_map_.find(key);
        if (it == tensor_map_.end()) {
            throw std::runtime_error("[FT][ERROR] Cannot find a tensor of name " + key + " in the tensor map");
        }
        return it->second;
    }
    const Tensor& at(const std::string& key) const
    {
        return const_cast<TensorMap*>(this)->at(key);
    }
    template<typename T>
    T getVal(const std::string& key) const
    {
        return at(key).getVal<T>();
    }
    template<typename T>
    T getVal(const std::string& key, T default_value) const
    {
        return isExist(key) ? at(key).getVal<T>() : default_value;
    }
    template<typename T>
    T* getPtr(const std::string& key, T* default_ptr = nullptr) const
    {
        return isExist(key) ? at(key).getPtr<T>() : default_ptr;
    }
    const std::unordered_map<std::string, Tensor>& getMap() const
    {
        return tensor_map_;
    }
};

class IAllocator {
public:
    virtual ~IAllocator() {}
    virtual void*        malloc(size_t size, const bool is_set_zero = true, bool is_host = false) = 0;
    virtual void         free(void** ptr, bool is_host = false) const                             = 0;
    virtual void         setStream(cudaStream_t stream)                                           = 0;
    virtual cudaStream_t returnStream()                                                           = 0;
    virtual void         memSet(void* ptr, const int val, const size_t size)                      = 0;
};

// cudaMalloc / cudaFree on the caller's stream; enough for tests and small hosts.
class CudaAllocator: public IAllocator {
    cudaStream_t stream_ = nullptr;

public:
    void* malloc(size_t size, const bool is_set_zero = true, bool is_host = false) override
    {
        void* p = nullptr;
        if (size == 0) {
            return nullptr;
        }
        cudaError_t e = is_host ? cudaMallocHost(&p, size) : cudaMalloc(&p, size);
        if (e != cudaSuccess) {
            throw std::runtime_error(std::string("[FT][ERROR] CUDA runtime error: ") + cudaGetErrorString(e));
        }
        if (is_set_zero) {
            if (is_host) {
                memset(p, 0, size);
            }
            else {
                cudaMemsetAsync(p, 0, size, stream_);
            }
        }
        return p;
    }
    void free(void** ptr, bool is_host = false) const override
    {
        if (ptr != nullptr && *ptr != nullptr) {
            is_host ? cudaFreeHost(*ptr) : cudaFree(*ptr);
            *ptr = nullptr;
        }
    }
    void setStream(cudaStream_t stream) override
    {
        stream_ = stream;
    }
    cudaStream_t returnStream() override
    {
        return stream_;
    }
    void memSet(void* ptr, const int val, const size_t size) override
    {
        cudaMemsetAsync(ptr, val, size, stream_);
    }
};

class cublasMMWrapper;  // passed through by callers, never used on this path

}  // namespace fastertransformer
