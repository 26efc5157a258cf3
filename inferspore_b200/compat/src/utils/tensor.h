// Tensor descriptors with the names, fields and methods of the InferSpore
// sources (reference: src/utils/tensor.h): Device, DataType, getTensorType<T>(),
// Tensor, TensorWrapper<T>, TensorMap.  They are non-owning views: `data` is a
// raw pointer the caller allocated and frees.
//
// One addition: numel(), the element count in 64 bits.  size() keeps the
// reference's `int` return type and therefore wraps for tensors of 2^31
// elements or more (a 32-layer KV cache has 2^35); the launch templates in
// src/kernels/ never call it.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>
#include <initializer_list>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <vector>

#include "src/utils/macro.h"
#include "src/utils/string_utils.h"

enum Device { CPU_PINNED, CPU, GPU };

enum DataType { FP32, FP16, INT8, INT32, BOOL, BYTES, UNSUPPORTED };

template <typename T>
DataType getTensorType() {
    using U = typename std::remove_cv<T>::type;
    if (std::is_same<U, float>::value) return FP32;
    if (std::is_same<U, half>::value) return FP16;
    if (std::is_same<U, int>::value) return INT32;
    if (std::is_same<U, int8_t>::value) return INT8;
    if (std::is_same<U, bool>::value) return BOOL;
    if (std::is_same<U, char>::value) return BYTES;
    return UNSUPPORTED;
}

template <typename T>
class TensorWrapper;

namespace ispore_compat {
inline const char* device_name(Device d) {
    switch (d) {
        case CPU: return "CPU";
        case CPU_PINNED: return "CPU_PINNED";
        case GPU: return "GPU";
    }
    return "?";
}
inline const char* dtype_name(DataType t) {
    switch (t) {
        case FP32: return "FP32";
        case FP16: return "FP16";
        case INT8: return "INT8";
        case INT32: return "INT32";
        case BOOL: return "BOOL";
        case BYTES: return "BYTES";
        default: return "UNSUPPORTED";
    }
}
inline int64_t shape_product(const std::vector<int>& shape) {
    if (shape.empty()) return 0;
    int64_t n = 1;
    for (int d : shape) n *= d;
    return n;
}
}  // namespace ispore_compat

struct Tensor {
    Device location;
    DataType dtype;
    std::vector<int> shape;

    Tensor() = default;
    Tensor(const Device location_, const DataType dtype_, const std::vector<int> shape_)
        : location(location_), dtype(dtype_), shape(shape_) {}
    virtual ~Tensor() = default;

    virtual int size() const { return static_cast<int>(ispore_compat::shape_product(shape)); }
    int64_t numel() const { return ispore_compat::shape_product(shape); }

    template <typename T>
    TensorWrapper<T>* as() {
        return static_cast<TensorWrapper<T>*>(this);
    }

    std::string DeviceString() const { return ispore_compat::device_name(location); }

    virtual std::string toString() const {
        return fmtstr("Tensor[where=%s, type=%s, shape=%s]", ispore_compat::device_name(location),
                      ispore_compat::dtype_name(dtype), vec2str(shape).c_str());
    }
};

template <typename T>
class TensorWrapper : public Tensor {
public:
    T* data = nullptr;

    TensorWrapper(Device location, DataType dtype, std::vector<int> shape) : Tensor(location, dtype, shape) {}

    TensorWrapper(Device location, DataType dtype, std::vector<int> shape, T* data)
        : Tensor(location, dtype, shape), data(data) {
        LLM_CHECK_WITH_INFO(getTensorType<T>() == dtype,
                            "when build TensorWrapper, the passed in data type should be same as dtype in params");
    }

    virtual int size() const {
        if (data == nullptr) return 0;
        return static_cast<int>(ispore_compat::shape_product(shape));
    }

    // Host reads: only legal for CPU-resident tensors (layer ids, decode step).
    inline T getVal(int id) const {
        LLM_CHECK(location == CPU);
        return data[id];
    }
    inline T getVal() const {
        LLM_CHECK(location == CPU);
        return getVal(0);
    }
    inline T* getPtr() const { return (T*)data; }
    inline T* getPtrByOffset(int offset) const { return (T*)data + offset; }

    virtual std::string toString() const {
        return fmtstr("Tensor[where=%s, type=%s, shape=%s, data=%p]", ispore_compat::device_name(location),
                      ispore_compat::dtype_name(dtype), vec2str(shape).c_str(), (void*)data);
    }
};

// Name -> Tensor* registry.  Invalid (empty) tensors are rejected on insert
// through the initializer-list constructor.
struct TensorMap {
    std::unordered_map<std::string, Tensor*> tensor_map_;

    TensorMap() = default;
    TensorMap(std::initializer_list<std::pair<std::string, Tensor*>> tensor_map) {
        for (auto& entry : tensor_map) {
            LLM_CHECK_WITH_INFO(isValid(entry.second),
                                fmtstr("%s is not a valid tensor, skipping insert into TensorMap",
                                       entry.first.c_str()));
            insert(entry.first, entry.second);
        }
    }
    TensorMap(const std::unordered_map<std::string, Tensor*>& tensor_map) {
        for (auto& entry : tensor_map)
            if (isValid(entry.second)) insert(entry.first, entry.second);
    }
    ~TensorMap() { tensor_map_.clear(); }

    inline size_t size() const { return tensor_map_.size(); }
    inline bool isExist(const std::string& key) const { return tensor_map_.find(key) != tensor_map_.end(); }
    inline bool isValid(const Tensor* tensor) { return tensor != nullptr && tensor->size() > 0; }
    inline void insert(const std::string& key, Tensor* value) { tensor_map_[key] = value; }
    inline void insert(std::pair<std::string, Tensor*> p) { tensor_map_.insert(p); }

    inline Tensor* at(const std::string& key) {
        LLM_CHECK_WITH_INFO(isExist(key), fmtstr("Cannot find a tensor of name %s in the tensor map (keys: %s)",
                                                 key.c_str(), vec2str(keys()).c_str()));
        return tensor_map_.at(key);
    }
    inline Tensor* operator[](const std::string& key) { return at(key); }

    std::vector<std::string> keys() const {
        std::vector<std::string> names;
        names.reserve(tensor_map_.size());
        for (auto& entry : tensor_map_) names.push_back(entry.first);
        return names;
    }
    std::string toString() {
        std::string out = "{";
        bool first = true;
        for (auto& entry : tensor_map_) {
            out += (first ? "" : ", ") + entry.first + ": " + entry.second->toString();
            first = false;
        }
        return out + "}";
    }
};
