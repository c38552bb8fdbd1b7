// TensorFlow binding: the six ops of libsbnet.so registered with the reference's exact interface
// (op names, attrs, inputs, outputs, host-memory placement), each GPU kernel forwarding to the C ABI
// of libsbnet_b200.so (include/sbnet_b200.h).
//
// Interface it reproduces (paths relative to sbnet_tensorflow/sbnet_ops/ of uber-research/sbnet):
//   ReduceMask                        reduce_mask.cc:100-110, GPU registration :236-247
//   SparseGather                      sparse_gather.cc:48-57,  GPU registration :229-238
//   SparseScatter / SparseScatterVar  sparse_gather.cc:242-268, GPU registration :374-387
//   CudaTimerStart / CudaTimerEnd     sparse_gather.cc:390-395, GPU registration :463-466
// Only the element type list differs: T is {float, half, bfloat16} for gather / scatter (the 16-bit
// types are additions; float graphs are unaffected).  There is no CPU kernel: this library is GPU only.
//
// Build (needs TensorFlow headers, which are not part of this repository's toolchain image):
//   g++ -std=c++17 -shared -fPIC sbnet_tf_ops.cc -o libsbnet.so \
//       $(python -c 'import tensorflow as tf; print(" ".join(tf.sysconfig.get_compile_flags()))') \
//       -I<repo>/include -L<repo>/sbnet_b200 -lsbnet_b200 \
//       $(python -c 'import tensorflow as tf; print(" ".join(tf.sysconfig.get_link_flags()))')
// This file is not compiled by the repository's own build; it is kept thin enough to be checked by
// reading it against the reference's Compute() methods.
#define EIGEN_USE_GPU
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/tensor_shape.h"

#include "sbnet_b200.h"

namespace {
using namespace tensorflow;
using GPUDevice = Eigen::GpuDevice;

// A length-2 int32 host tensor [H, W] (reduce_mask.cc:132-138, sparse_gather.cc:170-175).
Status ReadPair(const Tensor& t, const char* what, int* h, int* w)
{
    if (t.dims() != 1 || t.dim_size(0) != 2)
        return errors::InvalidArgument(what, " should be one-dimensional with shape[0] == 2.");
    const int32* p = t.flat<int32>().data();
    *h = p[0];
    *w = p[1];
    return Status::OK();
}

Status FromSbnet(int rc)
{
    if (rc == SBNET_OK)
        return Status::OK();
    if (rc < 0)
        return errors::InvalidArgument(sbnet_last_error());
    return errors::Internal(sbnet_last_error());
}

template <typename T> constexpr int SbnetType();
template <> constexpr int SbnetType<float>() { return SBNET_F32; }
template <> constexpr int SbnetType<Eigen::half>() { return SBNET_F16; }
template <> constexpr int SbnetType<bfloat16>() { return SBNET_BF16; }

void* StreamOf(OpKernelContext* ctx) { return (void*)ctx->eigen_device<GPUDevice>().stream(); }

struct Geometry {
    int szH, szW, strH, strW, offH, offW;
    Status Read(OpKernelContext* ctx, int first)
    {
        TF_RETURN_IF_ERROR(ReadPair(ctx->input(first), "dynamic_bsize", &szH, &szW));
        TF_RETURN_IF_ERROR(ReadPair(ctx->input(first + 1), "dynamic_bstride", &strH, &strW));
        return ReadPair(ctx->input(first + 2), "dynamic_boffset", &offH, &offW);
    }
};

class ReduceMaskGpu : public OpKernel {
public:
    explicit ReduceMaskGpu(OpKernelConstruction* c) : OpKernel(c)
    {
        OP_REQUIRES_OK(c, c->GetAttr("avgpool", &avgpool_));
        OP_REQUIRES_OK(c, c->GetAttr("tol", &tol_));
    }
    void Compute(OpKernelContext* ctx) override
    {
        const Tensor& mask = ctx->input(0);
        int cntH, cntW;
        Geometry g;
        OP_REQUIRES_OK(ctx, ReadPair(ctx->input(1), "dynamic_bcount", &cntH, &cntW));
        OP_REQUIRES_OK(ctx, g.Read(ctx, 2));
        const int N = mask.dim_size(0), H = mask.dim_size(1), W = mask.dim_size(2);
        Tensor* indices = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({(int64)N * cntH * cntW, 3}), &indices));
        Tensor scratch;   // per call, so concurrent Compute() calls never share it
        OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_INT32, TensorShape({SBNET_REDUCE_MASK_SCRATCH_INTS}), &scratch));
        Tensor* counts = nullptr;
        AllocatorAttributes host;
        host.set_on_host(true);
        host.set_gpu_compatible(true);   // pinned: the kernel writes the count straight into it
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, TensorShape({1}), &counts, host));
        OP_REQUIRES_OK(ctx, FromSbnet(sbnet_reduce_mask(
            mask.flat<float>().data(), N, H, W, tol_, avgpool_, g.offH, g.offW, g.szH, g.szW, g.strH, g.strW,
            cntH, cntW, indices->flat<int16>().data(), scratch.flat<int32>().data(),
            counts->flat<int32>().data(), /*flags=*/0, StreamOf(ctx))));
    }
private:
    float tol_ = 0;
    bool avgpool_ = false;
};

template <typename T> class SparseGatherGpu : public OpKernel {
public:
    explicit SparseGatherGpu(OpKernelConstruction* c) : OpKernel(c)
    {
        OP_REQUIRES_OK(c, c->GetAttr("transpose", &transpose_));
    }
    void Compute(OpKernelContext* ctx) override
    {
        const Tensor& x = ctx->input(0);
        OP_REQUIRES(ctx, x.dims() == 4, errors::InvalidArgument("x must be rank 4"));
        Geometry g;
        OP_REQUIRES_OK(ctx, g.Read(ctx, 3));
        const int nB = ctx->input(1).flat<int32>().data()[0];   // bin_counts lives in host memory
        const int N = x.dim_size(0), H = x.dim_size(1), W = x.dim_size(2), C = x.dim_size(3);
        const TensorShape shape = transpose_ ? TensorShape({nB, C, g.szH, g.szW})
                                             : TensorShape({nB, g.szH, g.szW, C});
        Tensor* y = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, shape, &y));
        OP_REQUIRES_OK(ctx, FromSbnet(sbnet_sparse_gather(
            x.flat<T>().data(), SbnetType<T>(), N, H, W, C, y->flat<T>().data(), g.offH, g.offW, g.szH,
            g.szW, g.strH, g.strW, nB, ctx->input(2).flat<int16>().data(), transpose_, StreamOf(ctx))));
    }
private:
    bool transpose_ = false;
};

template <typename T, bool kVar> class SparseScatterGpu : public OpKernel {
public:
    explicit SparseScatterGpu(OpKernelConstruction* c) : OpKernel(c)
    {
        OP_REQUIRES_OK(c, c->GetAttr("add", &add_));
        OP_REQUIRES_OK(c, c->GetAttr("transpose", &transpose_));
        OP_REQUIRES_OK(c, c->GetAttr("atomic", &atomic_));
    }
    void Compute(OpKernelContext* ctx) override
    {
        Tensor base = kVar ? ctx->mutable_input(3, false) : ctx->input(3);
        OP_REQUIRES(ctx, base.dims() == 4, errors::InvalidArgument("ybase must be rank 4"));
        Geometry g;
        OP_REQUIRES_OK(ctx, g.Read(ctx, 4));
        OP_REQUIRES(ctx, atomic_ || !add_ || (g.strH >= g.szH && g.strW >= g.szW),
                    errors::InvalidArgument("Only non-overlapping blocks are supported with add=True, atomic=False"));
        const int nB = ctx->input(1).flat<int32>().data()[0];
        const int N = base.dim_size(0), H = base.dim_size(1), W = base.dim_size(2), C = base.dim_size(3);
        T* out = nullptr;
        if (kVar) {
            ctx->forward_ref_input_to_ref_output(3, 0);
            out = base.flat<T>().data();
        } else {   // fresh output = copy of ybase, stream ordered (no synchronisation)
            Tensor* y = nullptr;
            OP_REQUIRES_OK(ctx, ctx->allocate_output(0, base.shape(), &y));
            out = y->flat<T>().data();
            OP_REQUIRES_OK(ctx, FromSbnet(sbnet_copy_tensor(out, base.flat<T>().data(),
                                                            base.NumElements() * sizeof(T), StreamOf(ctx))));
        }
        OP_REQUIRES_OK(ctx, FromSbnet(sbnet_sparse_scatter(
            ctx->input(0).flat<T>().data(), SbnetType<T>(), N, H, W, C, out, g.offH, g.offW, g.szH, g.szW,
            g.strH, g.strW, nB, ctx->input(2).flat<int16>().data(), add_, transpose_, atomic_, StreamOf(ctx))));
    }
private:
    bool add_ = false, transpose_ = false, atomic_ = false;
};

class TimerStartGpu : public OpKernel {
public:
    using OpKernel::OpKernel;
    void Compute(OpKernelContext* ctx) override
    {
        Tensor* out = nullptr;
        AllocatorAttributes host;
        host.set_on_host(true);
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({}), &out, host));
        int64_t handle = 0;
        OP_REQUIRES_OK(ctx, FromSbnet(sbnet_cuda_timer_start(&handle)));
        out->scalar<int64>()() = handle;
    }
};

class TimerEndGpu : public OpKernel {
public:
    using OpKernel::OpKernel;
    void Compute(OpKernelContext* ctx) override
    {
        Tensor* out = nullptr;
        AllocatorAttributes host;
        host.set_on_host(true);
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({}), &out, host));
        float ms = 0;
        OP_REQUIRES_OK(ctx, FromSbnet(sbnet_cuda_timer_end(ctx->input(0).scalar<int64>()(), &ms)));
        out->scalar<float>()() = ms;
    }
};
}  // namespace

REGISTER_OP("ReduceMask").Attr("T: {float}").Attr("tol: float").Attr("avgpool: bool = false")
    .Input("mask: T").Input("dynamic_bcount: int32").Input("dynamic_bsize: int32")
    .Input("dynamic_bstride: int32").Input("dynamic_boffset: int32")
    .Output("active_block_indices: int16").Output("bin_counts: int32");
REGISTER_OP("SparseGather").Attr("T: {float, half, bfloat16}").Attr("transpose: bool = false")
    .Input("x: T").Input("bin_counts: int32").Input("active_block_indices: int16")
    .Input("dynamic_bsize: int32").Input("dynamic_bstride: int32").Input("dynamic_boffset: int32")
    .Output("y: T");
REGISTER_OP("SparseScatterVar").Attr("T: {float, half, bfloat16}").Attr("add: bool").Attr("atomic: bool = false")
    .Attr("transpose: bool = false")
    .Input("x: T").Input("bin_counts: int32").Input("active_block_indices: int16").Input("ybase: Ref(T)")
    .Input("dynamic_bsize: int32").Input("dynamic_bstride: int32").Input("dynamic_boffset: int32")
    .Output("y: Ref(T)");
REGISTER_OP("SparseScatter").Attr("T: {float, half, bfloat16}").Attr("add: bool").Attr("atomic: bool = false")
    .Attr("transpose: bool = false")
    .Input("x: T").Input("bin_counts: int32").Input("active_block_indices: int16").Input("ybase: T")
    .Input("dynamic_bsize: int32").Input("dynamic_bstride: int32").Input("dynamic_boffset: int32")
    .Output("y: T");
REGISTER_OP("CudaTimerStart").Output("start_event: int64");
REGISTER_OP("CudaTimerEnd").Input("start_event: int64").Output("dt: float");

REGISTER_KERNEL_BUILDER(Name("ReduceMask").Device(DEVICE_GPU).TypeConstraint<float>("T")
                            .HostMemory("dynamic_bcount").HostMemory("dynamic_bsize")
                            .HostMemory("dynamic_bstride").HostMemory("dynamic_boffset")
                            .HostMemory("bin_counts"), ReduceMaskGpu);
#define SBNET_REGISTER_BLOCK_OPS(T)                                                                    \
    REGISTER_KERNEL_BUILDER(Name("SparseGather").Device(DEVICE_GPU).TypeConstraint<T>("T")             \
                                .HostMemory("bin_counts").HostMemory("dynamic_bsize")                  \
                                .HostMemory("dynamic_bstride").HostMemory("dynamic_boffset"),          \
                            SparseGatherGpu<T>);                                                       \
    REGISTER_KERNEL_BUILDER(Name("SparseScatter").Device(DEVICE_GPU).TypeConstraint<T>("T")            \
                                .HostMemory("bin_counts").HostMemory("dynamic_bsize")                  \
                                .HostMemory("dynamic_bstride").HostMemory("dynamic_boffset"),          \
                            SparseScatterGpu<T, false>);                                               \
    REGISTER_KERNEL_BUILDER(Name("SparseScatterVar").Device(DEVICE_GPU).TypeConstraint<T>("T")         \
                                .HostMemory("bin_counts").HostMemory("dynamic_bsize")                  \
                                .HostMemory("dynamic_bstride").HostMemory("dynamic_boffset"),          \
                            SparseScatterGpu<T, true>);
SBNET_REGISTER_BLOCK_OPS(float)
SBNET_REGISTER_BLOCK_OPS(Eigen::half)
SBNET_REGISTER_BLOCK_OPS(bfloat16)
REGISTER_KERNEL_BUILDER(Name("CudaTimerStart").Device(DEVICE_GPU).HostMemory("start_event"), TimerStartGpu);
REGISTER_KERNEL_BUILDER(Name("CudaTimerEnd").Device(DEVICE_GPU).HostMemory("dt").HostMemory("start_event"),
                        TimerEndGpu);
