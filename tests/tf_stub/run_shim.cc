// Drives the TensorFlow binding (sbnet_b200/csrc/tf_shim/sbnet_tf_ops.cc) without TensorFlow, on the
// stand-in API of tf_stub.h.  TEST INFRASTRUCTURE ONLY.
//   run_shim dump   prints every registered op and kernel as JSON (no CUDA call is made)
//   run_shim run    executes ReduceMask -> SparseGather -> SparseScatter[Var] and the timer ops through
//                   their OpKernel::Compute on a GPU and checks the results against the CPU checker
#include "../../sbnet_b200/csrc/tf_shim/sbnet_tf_ops.cc"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <numeric>

extern "C" {
void oracle_reduce_mask_op(const float*, int, int, int, float, int, int, int, int, int, int, int, int, int16_t*, int32_t*, int);
void oracle_sparse_gather_f32(const float*, int, int, int, int, float*, int, int, int, int, int, int, int, const int16_t*, int);
void oracle_sparse_scatter_f32(const float*, int, int, int, int, float*, int, int, int, int, int, int, int, const int16_t*, int, int, int);
}

using namespace tensorflow;

static DataType OutType(const std::string& spec, DataType T)
{
    const std::string t = spec.substr(spec.find(':') + 1);
    if (t.find("int16") != std::string::npos) return DT_INT16;
    if (t.find("int32") != std::string::npos) return DT_INT32;
    if (t.find("int64") != std::string::npos) return DT_INT64;
    if (t.find("float") != std::string::npos) return DT_FLOAT;
    return T;
}

static Status g_last;

struct Runner {
    cudaStream_t stream = nullptr;
    Status Run(const std::string& op, DataType T, const std::map<std::string, AttrValue>& attrs,
               std::vector<Tensor> inputs, std::vector<Tensor>* outputs)
    {
        const OpDef* def = nullptr;
        for (auto& d : Registry::Get().ops) if (d.name == op) def = &d;
        const KernelDef* k = nullptr;
        for (auto& kd : Registry::Get().kernels) if (kd.op == op && (!kd.typed || kd.type == T)) k = &kd;
        if (!def || !k) return errors::Internal("no registration for ", op);
        OpKernelConstruction c;
        c.attrs = attrs;
        std::unique_ptr<OpKernel> kernel(k->factory(&c));
        if (!c.status.ok()) return c.status;
        OpKernelContext ctx;
        ctx.inputs = inputs;
        ctx.device.stream_ = stream;
        for (auto& o : def->outputs) ctx.output_types.push_back(OutType(o, T));
        ctx.outputs.resize(def->outputs.size());   // fixed size: kernels keep pointers into it
        kernel->Compute(&ctx);
        g_last = ctx.status;
        if (!ctx.status.ok()) return ctx.status;
        *outputs = ctx.outputs;
        return Status::OK();
    }
};

static Tensor HostPair(int a, int b)
{
    Tensor t(DT_INT32, TensorShape({2}), true);
    t.flat<int32>().data()[0] = a;
    t.flat<int32>().data()[1] = b;
    return t;
}
static Tensor DevFloat(const std::vector<float>& v, std::initializer_list<int64> shape)
{
    Tensor t(DT_FLOAT, TensorShape(shape), false);
    cudaMemcpy(t.raw(), v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return t;
}
template <typename T> static std::vector<T> ToHost(const Tensor& t, size_t n)
{
    std::vector<T> v(n);
    if (t.on_host()) memcpy(v.data(), t.raw(), n * sizeof(T)); else cudaMemcpy(v.data(), t.raw(), n * sizeof(T), cudaMemcpyDeviceToHost);
    return v;
}
static AttrValue B(bool b) { AttrValue a; a.b = b; return a; }
static AttrValue F(float f) { AttrValue a; a.f = f; return a; }
#define CHECK_TRUE(x) do { if (!(x)) { printf("FAIL line %d: %s [%d %s]\n", __LINE__, #x, g_last.code(), g_last.error_message().c_str()); return 1; } } while (0)

static void PrintList(const std::vector<std::string>& v)
{
    printf("[");
    for (size_t i = 0; i < v.size(); ++i) printf("%s\"%s\"", i ? ", " : "", v[i].c_str());
    printf("]");
}

static int Dump()
{
    printf("{\"ops\": [");
    bool first = true;
    for (auto& d : Registry::Get().ops) {
        printf("%s{\"name\": \"%s\", \"attrs\": ", first ? "" : ", ", d.name.c_str());
        PrintList(d.attrs);
        printf(", \"inputs\": ");
        PrintList(d.inputs);
        printf(", \"outputs\": ");
        PrintList(d.outputs);
        printf("}");
        first = false;
    }
    printf("], \"kernels\": [");
    first = true;
    for (auto& k : Registry::Get().kernels) {
        printf("%s{\"op\": \"%s\", \"device\": \"%s\", \"type\": %d, \"host_memory\": ", first ? "" : ", ", k.op.c_str(),
               k.device.c_str(), k.typed ? (int)k.type : -1);
        PrintList(k.host_memory);
        printf("}");
        first = false;
    }
    printf("]}\n");
    return 0;
}

static int RunAll()
{
    const int N = 2, H = 40, W = 56, C = 32, BS = 10, ST = 8, OFF = -1;
    const int bch = 1 + (H - OFF - 1) / ST, bcw = 1 + (W - OFF - 1) / ST;
    std::vector<float> mask((size_t)N * H * W), x((size_t)N * H * W * C);
    uint32_t s = 12345;
    auto rnd = [&]() { s = s * 1664525u + 1013904223u; return (s >> 8) * (1.0f / 16777216.0f); };
    for (int n = 0; n < N; ++n)
        for (int h = 0; h < H; ++h)
            for (int w = 0; w < W; ++w) mask[((size_t)n * H + h) * W + w] = ((h / 8 * 7 + w / 8 * 3 + n) % 5 == 0) ? 1.0f : 0.0f;
    for (auto& v : x) v = rnd() * 2 - 1;

    Runner r;
    cudaStreamCreate(&r.stream);
    std::vector<Tensor> out;
    // ---- ReduceMask
    Status st = r.Run("ReduceMask", DT_FLOAT, {{"tol", F(0.5f)}, {"avgpool", B(false)}},
                      {DevFloat(mask, {N, H, W, 1}), HostPair(bch, bcw), HostPair(BS, BS), HostPair(ST, ST), HostPair(OFF, OFF)}, &out);
    CHECK_TRUE(st.ok());
    CHECK_TRUE(out[0].dims() == 2 && out[0].dim_size(0) == N * bch * bcw && out[0].dim_size(1) == 3 && out[1].on_host());
    Tensor idxT = out[0], cntT = out[1];
    const int nb = cntT.flat<int32>().data()[0];
    std::vector<int16_t> oidx((size_t)N * bch * bcw * 3);
    int32_t ocnt = 0;
    oracle_reduce_mask_op(mask.data(), N, H, W, 0.5f, OFF, OFF, BS, BS, ST, ST, bch, bcw, oidx.data(), &ocnt, 0);
    CHECK_TRUE(nb == ocnt && nb > 4);
    std::vector<int16_t> gidx = ToHost<int16_t>(idxT, (size_t)nb * 3);
    std::vector<int> order(nb);
    std::iota(order.begin(), order.end(), 0);
    auto key = [&](int i) { return (gidx[i * 3] * bch + gidx[i * 3 + 1]) * bcw + gidx[i * 3 + 2]; };
    std::sort(order.begin(), order.end(), [&](int a, int b) { return key(a) < key(b); });
    for (int i = 0; i < nb; ++i)
        for (int k = 0; k < 3; ++k) CHECK_TRUE(gidx[order[i] * 3 + k] == oidx[i * 3 + k]);
    // bad geometry tensor -> InvalidArgument
    Tensor bad(DT_INT32, TensorShape({3}), true);
    st = r.Run("ReduceMask", DT_FLOAT, {{"tol", F(0.5f)}, {"avgpool", B(false)}},
               {DevFloat(mask, {N, H, W, 1}), bad, HostPair(BS, BS), HostPair(ST, ST), HostPair(OFF, OFF)}, &out);
    CHECK_TRUE(st.code() == 3);

    const size_t blk = (size_t)BS * BS * C;
    Tensor xT = DevFloat(x, {N, H, W, C});
    for (int tr = 0; tr < 2; ++tr) {
        // ---- SparseGather
        st = r.Run("SparseGather", DT_FLOAT, {{"transpose", B(tr)}}, {xT, cntT, idxT, HostPair(BS, BS), HostPair(ST, ST), HostPair(OFF, OFF)}, &out);
        CHECK_TRUE(st.ok());
        CHECK_TRUE(out[0].dim_size(0) == nb && out[0].dim_size(1) == (tr ? C : BS) && out[0].dim_size(3) == (tr ? BS : C));
        Tensor stackT = out[0];
        std::vector<float> got = ToHost<float>(stackT, nb * blk), exp(nb * blk);
        oracle_sparse_gather_f32(x.data(), N, H, W, C, exp.data(), OFF, OFF, BS, BS, ST, ST, nb, gidx.data(), tr);
        CHECK_TRUE(memcmp(got.data(), exp.data(), got.size() * 4) == 0);
        // ---- SparseScatter (fresh output = copy of ybase, overwrite with gathered values)
        std::vector<float> base(x.size(), 10.0f);
        Tensor baseT = DevFloat(base, {N, H, W, C});
        st = r.Run("SparseScatter", DT_FLOAT, {{"add", B(false)}, {"atomic", B(false)}, {"transpose", B(tr)}},
                   {stackT, cntT, idxT, baseT, HostPair(BS, BS), HostPair(ST, ST), HostPair(OFF, OFF)}, &out);
        CHECK_TRUE(st.ok());
        std::vector<float> y = ToHost<float>(out[0], x.size()), ey = base;
        oracle_sparse_scatter_f32(exp.data(), N, H, W, C, ey.data(), OFF, OFF, BS, BS, ST, ST, nb, gidx.data(), 0, tr, 0);
        CHECK_TRUE(memcmp(y.data(), ey.data(), y.size() * 4) == 0);
        std::vector<float> stillBase = ToHost<float>(baseT, x.size());
        CHECK_TRUE(stillBase[0] == 10.0f && stillBase.back() == 10.0f);   // the non-Var op must not touch ybase
        // ---- SparseScatterVar, atomic add over the overlapping halos, in place
        st = r.Run("SparseScatterVar", DT_FLOAT, {{"add", B(true)}, {"atomic", B(true)}, {"transpose", B(tr)}},
                   {stackT, cntT, idxT, baseT, HostPair(BS, BS), HostPair(ST, ST), HostPair(OFF, OFF)}, &out);
        CHECK_TRUE(st.ok() && out[0].raw() == baseT.raw());
        y = ToHost<float>(baseT, x.size());
        ey = base;
        oracle_sparse_scatter_f32(exp.data(), N, H, W, C, ey.data(), OFF, OFF, BS, BS, ST, ST, nb, gidx.data(), 1, tr, 1);
        for (size_t i = 0; i < y.size(); ++i) CHECK_TRUE(std::fabs(y[i] - ey[i]) <= 4e-6f * std::max(1.0f, std::fabs(ey[i])));
        // ---- add without atomics on overlapping blocks is rejected like in the reference
        st = r.Run("SparseScatterVar", DT_FLOAT, {{"add", B(true)}, {"atomic", B(false)}, {"transpose", B(tr)}},
                   {stackT, cntT, idxT, baseT, HostPair(BS, BS), HostPair(ST, ST), HostPair(OFF, OFF)}, &out);
        CHECK_TRUE(st.code() == 3 && st.error_message().find("non-overlapping") != std::string::npos);
    }
    // ---- timers
    st = r.Run("CudaTimerStart", DT_FLOAT, {}, {}, &out);
    CHECK_TRUE(st.ok());
    Tensor h = out[0];
    st = r.Run("CudaTimerEnd", DT_FLOAT, {}, {h}, &out);
    CHECK_TRUE(st.ok() && out[0].scalar<float>()() >= 0.0f);
    printf("PASS %d blocks\n", nb);
    return 0;
}

int main(int argc, char** argv)
{
    if (argc > 1 && std::string(argv[1]) == "dump") return Dump();
    return RunAll();
}
