// A very small stand-in for the parts of the TensorFlow C++ op API that the binding in
// sbnet_b200/csrc/tf_shim/sbnet_tf_ops.cc uses.  TEST INFRASTRUCTURE ONLY: it lets the binding be
// compiled and its OpKernels be executed without TensorFlow (which is not installed here), so that
// the registrations can be compared with the reference's and Compute() can be run on a GPU against
// the CPU checker.  Tensors are plain buffers; "GPU" tensors live in cudaMalloc'ed memory.
#pragma once
#include <cuda_runtime_api.h>

#include <cstdint>
#include <functional>
#include <initializer_list>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace Eigen {
struct half { uint16_t x; };
struct GpuDevice {
    cudaStream_t stream_ = nullptr;
    cudaStream_t stream() const { return stream_; }
};
}  // namespace Eigen

namespace tensorflow {
typedef int16_t int16;
typedef int32_t int32;
typedef long long int64;
struct bfloat16 { uint16_t x; };
enum DataType { DT_FLOAT, DT_HALF, DT_INT16, DT_INT32, DT_INT64, DT_BFLOAT16 };
inline size_t DataTypeSize(DataType t)
{
    return t == DT_FLOAT ? 4 : (t == DT_HALF || t == DT_BFLOAT16 || t == DT_INT16) ? 2 : t == DT_INT32 ? 4 : 8;
}
template <typename T> struct DataTypeOf;
template <> struct DataTypeOf<float> { static const DataType v = DT_FLOAT; };
template <> struct DataTypeOf<Eigen::half> { static const DataType v = DT_HALF; };
template <> struct DataTypeOf<bfloat16> { static const DataType v = DT_BFLOAT16; };
template <> struct DataTypeOf<int16> { static const DataType v = DT_INT16; };
template <> struct DataTypeOf<int32> { static const DataType v = DT_INT32; };
template <> struct DataTypeOf<int64> { static const DataType v = DT_INT64; };
static const char* const DEVICE_GPU = "GPU";

class Status {
public:
    Status() {}
    Status(int code, const std::string& m) : code_(code), msg_(m) {}
    static Status OK() { return Status(); }
    bool ok() const { return code_ == 0; }
    int code() const { return code_; }
    const std::string& error_message() const { return msg_; }
private:
    int code_ = 0;
    std::string msg_;
};
namespace errors {
inline void Cat(std::ostringstream&) {}
template <typename A, typename... R> void Cat(std::ostringstream& o, const A& a, const R&... r) { o << a; Cat(o, r...); }
template <typename... A> Status InvalidArgument(const A&... a) { std::ostringstream o; Cat(o, a...); return Status(3, o.str()); }
template <typename... A> Status Internal(const A&... a) { std::ostringstream o; Cat(o, a...); return Status(13, o.str()); }
}  // namespace errors
#define TF_RETURN_IF_ERROR(expr) do { ::tensorflow::Status _s = (expr); if (!_s.ok()) return _s; } while (0)

class TensorShape {
public:
    TensorShape() {}
    TensorShape(std::initializer_list<int64> d) : dims_(d) {}
    int dims() const { return (int)dims_.size(); }
    int64 dim_size(int i) const { return dims_[i]; }
    int64 num_elements() const { int64 n = 1; for (int64 d : dims_) n *= d; return n; }
    std::vector<int64> dims_;
};

struct AllocatorAttributes {
    bool on_host = false, gpu_compatible = false;
    void set_on_host(bool v) { on_host = v; }
    void set_gpu_compatible(bool v) { gpu_compatible = v; }
};

// A buffer with a shape.  Device tensors own cudaMalloc'ed memory, host tensors pinned memory.
class Tensor {
public:
    Tensor() {}
    Tensor(DataType t, const TensorShape& s, bool on_host) : dtype_(t), shape_(s), on_host_(on_host)
    {
        size_t bytes = (size_t)s.num_elements() * DataTypeSize(t);
        if (bytes == 0) bytes = 16;
        void* p = nullptr;
        if (on_host) cudaMallocHost(&p, bytes); else cudaMalloc(&p, bytes);
        const bool h = on_host;
        buf_ = std::shared_ptr<void>(p, [h](void* q) { if (h) cudaFreeHost(q); else cudaFree(q); });
    }
    int dims() const { return shape_.dims(); }
    int64 dim_size(int i) const { return shape_.dim_size(i); }
    int64 NumElements() const { return shape_.num_elements(); }
    const TensorShape& shape() const { return shape_; }
    DataType dtype() const { return dtype_; }
    bool on_host() const { return on_host_; }
    void* raw() const { return buf_.get(); }
    template <typename T> struct Flat {
        T* p;
        T* data() const { return p; }
    };
    template <typename T> Flat<T> flat() const { return Flat<T>{static_cast<T*>(buf_.get())}; }
    template <typename T> struct Scalar {
        T* p;
        T& operator()() const { return *p; }
    };
    template <typename T> Scalar<T> scalar() const { return Scalar<T>{static_cast<T*>(buf_.get())}; }
private:
    DataType dtype_ = DT_FLOAT;
    TensorShape shape_;
    bool on_host_ = false;
    std::shared_ptr<void> buf_;
};

struct AttrValue { bool b = false; float f = 0; };

class OpKernelConstruction {
public:
    std::map<std::string, AttrValue> attrs;
    Status status;
    Status GetAttr(const std::string& n, bool* v) { auto it = attrs.find(n); if (it == attrs.end()) return errors::InvalidArgument("no attr ", n); *v = it->second.b; return Status::OK(); }
    Status GetAttr(const std::string& n, float* v) { auto it = attrs.find(n); if (it == attrs.end()) return errors::InvalidArgument("no attr ", n); *v = it->second.f; return Status::OK(); }
    void CtxFailure(const Status& s) { status = s; }
};

class OpKernelContext {
public:
    std::vector<Tensor> inputs;
    std::vector<Tensor> outputs;
    std::vector<DataType> output_types;   // from the op registration
    Eigen::GpuDevice device;
    Status status;
    int forwarded_input = -1;
    const Tensor& input(int i) { return inputs[i]; }
    Tensor mutable_input(int i, bool) { return inputs[i]; }
    Status allocate_output(int i, const TensorShape& s, Tensor** out, AllocatorAttributes a = AllocatorAttributes())
    {
        outputs.at(i) = Tensor(output_types.at(i), s, a.on_host);   // `outputs` is pre-sized by the driver
        *out = &outputs[i];
        return Status::OK();
    }
    Status allocate_temp(DataType t, const TensorShape& s, Tensor* out) { *out = Tensor(t, s, false); return Status::OK(); }
    void forward_ref_input_to_ref_output(int in, int out) { forwarded_input = in; outputs.at(out) = inputs[in]; }
    template <typename D> const D& eigen_device() const { return device; }
    void CtxFailure(const Status& s) { status = s; }
};

class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction*) {}
    virtual ~OpKernel() {}
    virtual void Compute(OpKernelContext* ctx) = 0;
};

#define OP_REQUIRES(CTX, EXP, STATUS) do { if (!(EXP)) { (CTX)->CtxFailure((STATUS)); return; } } while (0)
#define OP_REQUIRES_OK(CTX, ...) do { ::tensorflow::Status _s(__VA_ARGS__); if (!_s.ok()) { (CTX)->CtxFailure(_s); return; } } while (0)

// ---- registries ----------------------------------------------------------------------------------
struct OpDef {
    std::string name;
    std::vector<std::string> attrs, inputs, outputs;
    OpDef& Attr(const std::string& s) { attrs.push_back(s); return *this; }
    OpDef& Input(const std::string& s) { inputs.push_back(s); return *this; }
    OpDef& Output(const std::string& s) { outputs.push_back(s); return *this; }
};
struct KernelDef {
    std::string op, device, type_attr;
    DataType type = DT_FLOAT;
    bool typed = false;
    std::vector<std::string> host_memory;
    KernelDef& Device(const char* d) { device = d; return *this; }
    template <typename T> KernelDef& TypeConstraint(const char* attr) { type_attr = attr; type = DataTypeOf<T>::v; typed = true; return *this; }
    KernelDef& HostMemory(const char* a) { host_memory.push_back(a); return *this; }
    std::function<OpKernel*(OpKernelConstruction*)> factory;
};
inline KernelDef Name(const char* op) { KernelDef k; k.op = op; return k; }
struct Registry {
    std::vector<OpDef> ops;
    std::vector<KernelDef> kernels;
    static Registry& Get() { static Registry r; return r; }
};
struct OpRegistrar { OpRegistrar(const OpDef& d) { Registry::Get().ops.push_back(d); } };
struct KernelRegistrar {
    KernelRegistrar(KernelDef d, std::function<OpKernel*(OpKernelConstruction*)> f) { d.factory = f; Registry::Get().kernels.push_back(d); }
};
inline OpDef MakeOp(const char* n) { OpDef d; d.name = n; return d; }
#define TF_STUB_CAT2(a, b) a##b
#define TF_STUB_CAT(a, b) TF_STUB_CAT2(a, b)
#define REGISTER_OP(NAME) static ::tensorflow::OpRegistrar TF_STUB_CAT(op_registrar_, __COUNTER__) = ::tensorflow::MakeOp(NAME)
#define REGISTER_KERNEL_BUILDER(BUILDER, ...) \
    static ::tensorflow::KernelRegistrar TF_STUB_CAT(kernel_registrar_, __COUNTER__)( \
        BUILDER, [](::tensorflow::OpKernelConstruction* c) -> ::tensorflow::OpKernel* { return new __VA_ARGS__(c); })
}  // namespace tensorflow
