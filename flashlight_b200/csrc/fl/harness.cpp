/*
 * Harness that runs B200AutogradExtension behind real fl::Tensor objects, without ArrayFire.
 *
 * It registers the extension for the `Stub` backend slot exactly the way the cuDNN / oneDNN
 * ones are registered (flashlight/fl/autograd/tensor/AutogradExtensionBackends.h:28-42), makes
 * B200Tensor the default tensor type (flashlight/fl/tensor/TensorAdapter.h:358-365) and exposes
 * a few extern "C" calls that take HOST buffers, wrap them as fl::Tensor, and call the
 * reference's own dispatchers fl::detail::conv2d / conv2dBackwardData / ... / rnnBackward
 * (flashlight/fl/autograd/tensor/AutogradOps.cpp:146-361), which reach the extension through
 * TensorBackend::getExtension (flashlight/fl/tensor/TensorBackend.h:283-300).  So the path
 * Tensor -> dispatcher -> registry -> B200AutogradExtension -> DevicePtr / relativeSync -> C ABI
 * -> kernels runs end to end; tests/test_fl_harness_gpu.py checks the results against the
 * oracle.  The reference's tensor / runtime / autograd-ops sources are compiled in place from
 * the checkout by build_harness.py; nothing of them is copied here.
 *
 * Extents are fl order (dimension 0 fastest); every tensor is f32.  A null pointer stands for
 * an empty fl::Tensor.  Return value: 0 ok, 1 std::invalid_argument, 2 any other exception;
 * flb200_fl_last_error() has the message.
 */
#include <cstring>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "B200AutogradExtension.h"
#include "B200Tensor.h"
#include "flashlight/fl/common/DynamicBenchmark.h"
#include "flashlight/fl/autograd/tensor/AutogradOps.h"
#include "flashlight/fl/tensor/TensorBase.h"
#include "flashlight/fl/tensor/TensorExtension.h"

namespace fl {
FL_REGISTER_TENSOR_EXTENSION(B200AutogradExtension, Stub);
// The Tensor-level half of fl::distributed, defined in B200DistributedBackend.cpp with the
// signatures of flashlight/fl/distributed/DistributedApi.h:33-136.
void distributedInit(
    DistributedInit initMethod,
    int worldRank,
    int worldSize,
    const std::unordered_map<std::string, std::string>& params);
int getWorldRank();
int getWorldSize();
void allReduce(Tensor& arr, bool async);
void allReduceMultiple(std::vector<Tensor*> arrs, bool async, bool contiguous);
void syncDistributed();
}

namespace {

thread_local std::string g_error;

template <typename F>
int guarded(F&& f) {
  try {
    f();
    // a bounded device wait that ran out leaves partial results: make it an error here
    auto& ext = fl::B200Backend::getInstance().getExtension<fl::AutogradExtension>();
    static_cast<fl::B200AutogradExtension&>(ext).checkDeviceWaits();
    return 0;
  } catch (const std::invalid_argument& e) {
    g_error = e.what();
    return 1;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 2;
  }
}

fl::Tensor in(const float* p, std::vector<fl::Dim> dims) {
  if (!p) {
    return fl::Tensor();
  }
  return fl::Tensor::fromBuffer(fl::Shape(dims), p, fl::Location::Host);
}

void out(const fl::Tensor& t, float* p) {
  if (p && !t.isEmpty()) {
    t.host(p);
  }
}

using Payload = std::shared_ptr<fl::detail::AutogradPayload>;
Payload payload(void* h) {
  return h ? *static_cast<Payload*>(h) : nullptr;
}

} // namespace

extern "C" {

int flb200_fl_init(void) {
  return guarded([] { fl::setDefaultTensorType<fl::B200Tensor>(); });
}

const char* flb200_fl_last_error(void) {
  return g_error.c_str();
}

// 1 when fl::Tensor objects are B200Tensors whose backend hands out B200AutogradExtension.
int flb200_fl_registered(void) {
  try {
    fl::Tensor t({2}, fl::dtype::f32);
    auto& ext = t.backend().getExtension<fl::AutogradExtension>();
    return dynamic_cast<fl::B200AutogradExtension*>(&ext) != nullptr &&
            t.backendType() == fl::TensorBackendType::Stub
        ? 1
        : 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 0;
  }
}

void* flb200_fl_payload_new(void) {
  return new Payload(std::make_shared<fl::detail::AutogradPayload>());
}
void flb200_fl_payload_free(void* h) {
  delete static_cast<Payload*>(h);
}

int flb200_fl_conv2d(
    const float* x, const float* w, const float* bias, float* y, int W, int H, int C, int N,
    int kW, int kH, int Cout, int Wo, int Ho, int sx, int sy, int px, int py, int dx, int dy,
    int groups, void* pl) {
  return guarded([&] {
    auto r = fl::detail::conv2d(
        in(x, {W, H, C, N}), in(w, {kW, kH, C / groups, Cout}), in(bias, {1, 1, Cout, 1}), sx, sy,
        px, py, dx, dy, groups, payload(pl));
    if (r.dim(0) != Wo || r.dim(1) != Ho || r.dim(2) != Cout || r.dim(3) != N) {
      throw std::runtime_error("conv2d: unexpected output shape");
    }
    out(r, y);
  });
}

int flb200_fl_conv2d_backward_data(
    const float* gy, const float* x, const float* w, float* gx, int W, int H, int C, int N, int kW,
    int kH, int Cout, int Wo, int Ho, int sx, int sy, int px, int py, int dx, int dy, int groups,
    void* pl) {
  return guarded([&] {
    auto r = fl::detail::conv2dBackwardData(
        in(gy, {Wo, Ho, Cout, N}), in(x, {W, H, C, N}), in(w, {kW, kH, C / groups, Cout}), sx, sy,
        px, py, dx, dy, groups, nullptr, payload(pl));
    out(r, gx);
  });
}

int flb200_fl_conv2d_backward_filter_bias(
    const float* gy, const float* x, const float* w, const float* bias, float* gw, float* gb,
    int W, int H, int C, int N, int kW, int kH, int Cout, int Wo, int Ho, int sx, int sy, int px,
    int py, int dx, int dy, int groups, void* pl) {
  return guarded([&] {
    auto r = fl::detail::conv2dBackwardFilterBias(
        in(gy, {Wo, Ho, Cout, N}), in(x, {W, H, C, N}), in(w, {kW, kH, C / groups, Cout}),
        in(bias, {1, 1, Cout, 1}), sx, sy, px, py, dx, dy, groups, nullptr, nullptr, payload(pl));
    out(r.first, gw);
    if (bias && r.second.isEmpty()) {
      throw std::runtime_error("conv2dBackwardFilterBias: bias gradient missing");
    }
    if (!bias && !r.second.isEmpty()) {
      throw std::runtime_error("conv2dBackwardFilterBias: bias gradient for an absent bias");
    }
    out(r.second, gb);
  });
}

int flb200_fl_pool2d(
    const float* x, float* y, int W, int H, int C, int N, int Wo, int Ho, int wx, int wy, int sx,
    int sy, int px, int py, int mode, void* pl) {
  return guarded([&] {
    auto r = fl::detail::pool2d(
        in(x, {W, H, C, N}), wx, wy, sx, sy, px, py, static_cast<fl::PoolingMode>(mode),
        payload(pl));
    if (r.dim(0) != Wo || r.dim(1) != Ho) {
      throw std::runtime_error("pool2d: unexpected output shape");
    }
    out(r, y);
  });
}

int flb200_fl_pool2d_backward(
    const float* gy, const float* x, const float* y, float* gx, int W, int H, int C, int N, int Wo,
    int Ho, int wx, int wy, int sx, int sy, int px, int py, int mode, void* pl) {
  return guarded([&] {
    auto r = fl::detail::pool2dBackward(
        in(gy, {Wo, Ho, C, N}), in(x, {W, H, C, N}), in(y, {Wo, Ho, C, N}), wx, wy, sx, sy, px, py,
        static_cast<fl::PoolingMode>(mode), payload(pl));
    out(r, gx);
  });
}

// shape: ndim extents in fl order; axes: fl axes; channels = product of the extents at axes.
// running_mean / running_var are read and written back when given.
int flb200_fl_batchnorm(
    const float* x, const float* weight, const float* bias, float* running_mean,
    float* running_var, float* save_mean, float* save_var, float* y, const int* shape, int ndim,
    const int* axes, int naxes, int channels, int train, double momentum, double epsilon) {
  return guarded([&] {
    std::vector<fl::Dim> dims(shape, shape + ndim);
    std::vector<int> ax(axes, axes + naxes);
    fl::Tensor rm = in(running_mean, {channels}), rv = in(running_var, {channels});
    fl::Tensor sm, sv;
    auto r = fl::detail::batchnorm(
        sm, sv, in(x, dims), in(weight, {channels}), in(bias, {channels}), rm, rv, ax, train != 0,
        momentum, epsilon, nullptr);
    out(r, y);
    out(sm, save_mean);
    out(sv, save_var);
    out(rm, running_mean);
    out(rv, running_var);
  });
}

int flb200_fl_batchnorm_backward(
    const float* gy, const float* save_mean, const float* save_var, const float* x,
    const float* weight, float* gx, float* gw, float* gb, const int* shape, int ndim,
    const int* axes, int naxes, int channels, int train, float epsilon) {
  return guarded([&] {
    std::vector<fl::Dim> dims(shape, shape + ndim);
    std::vector<int> ax(axes, axes + naxes);
    auto r = fl::detail::batchnormBackward(
        in(gy, dims), in(save_mean, {channels}), in(save_var, {channels}), in(x, dims),
        in(weight, {channels}), ax, train != 0, epsilon, nullptr);
    out(std::get<0>(r), gx);
    out(std::get<1>(r), gw);
    out(std::get<2>(r), gb);
  });
}

int flb200_fl_rnn(
    const float* x, const float* hx, const float* cx, const float* w, long long nparams, float* y,
    float* hy, float* cy, int I, int B, int T, int hidden, int layers, int mode, int bidirectional,
    float dropout, void* pl) {
  return guarded([&] {
    const int dirs = bidirectional ? 2 : 1;
    auto r = fl::detail::rnn(
        in(x, {I, B, T}), in(hx, {hidden, B, layers * dirs}), in(cx, {hidden, B, layers * dirs}),
        in(w, {nparams}), hidden, layers, static_cast<fl::RnnMode>(mode), bidirectional != 0,
        dropout, payload(pl));
    out(std::get<0>(r), y);
    out(std::get<1>(r), hy);
    out(std::get<2>(r), cy);
  });
}

int flb200_fl_rnn_backward(
    const float* x, const float* hx, const float* cx, const float* w, long long nparams,
    const float* y, const float* gy, const float* ghy, const float* gcy, float* gx, float* ghx,
    float* gcx, float* gw, int I, int B, int T, int hidden, int layers, int mode,
    int bidirectional, float dropout, void* pl) {
  return guarded([&] {
    const int dirs = bidirectional ? 2 : 1;
    auto grads = std::make_shared<fl::detail::RNNGradData>();
    grads->dy = in(gy, {hidden * dirs, B, T});
    grads->dhy = in(ghy, {hidden, B, layers * dirs});
    grads->dcy = in(gcy, {hidden, B, layers * dirs});
    auto r = fl::detail::rnnBackward(
        in(x, {I, B, T}), in(hx, {hidden, B, layers * dirs}), in(cx, {hidden, B, layers * dirs}),
        in(w, {nparams}), grads, in(y, {hidden * dirs, B, T}), layers, hidden,
        static_cast<fl::RnnMode>(mode), bidirectional != 0, dropout, payload(pl));
    out(std::get<0>(r), gx);
    out(std::get<1>(r), ghx);
    out(std::get<2>(r), gcx);
    out(std::get<3>(r), gw);
  });
}

// ---- f16 activations: one bottleneck-style chain conv2d -> batchnorm -> pool2d and its
// gradients on f16 fl::Tensor objects (f32 host buffers in and out; batch-norm parameters f32) ----
int flb200_fl_half_chain(
    const float* x, const float* w, const float* gamma, const float* beta, const float* gy,
    float* y, float* gx, float* gw, float* ggamma, float* gbeta, int W, int H, int C, int N,
    int k, int Cout, int pad) {
  return guarded([&] {
    const auto f16 = fl::dtype::f16;
    auto& ext = fl::Tensor().backend().getExtension<fl::AutogradExtension>();
    if (!ext.isDataTypeSupported(f16)) {
      throw std::runtime_error("the extension does not report f16 as supported");
    }
    auto tx = in(x, {W, H, C, N}).astype(f16);
    auto tw = in(w, {k, k, C, Cout}).astype(f16);
    auto tg = in(gamma, {Cout});
    auto tb = in(beta, {Cout});
    auto pc = std::make_shared<fl::detail::AutogradPayload>();
    auto pp = std::make_shared<fl::detail::AutogradPayload>();
    auto c = fl::detail::conv2d(tx, tw, fl::Tensor(), 1, 1, pad, pad, 1, 1, 1, pc);
    fl::Tensor sm, sv, rm, rv;
    auto b = fl::detail::batchnorm(sm, sv, c, tg, tb, rm, rv, {2}, true, 0.1, 1e-5, nullptr);
    auto p = fl::detail::pool2d(b, 2, 2, 2, 2, 0, 0, fl::PoolingMode::AVG_INCLUDE_PADDING, pp);
    if (c.type() != f16 || b.type() != f16 || p.type() != f16 || sm.type() != fl::dtype::f32) {
      throw std::runtime_error("unexpected result types in the f16 chain");
    }
    out(p.astype(fl::dtype::f32), y);
    auto tgy = in(gy, {p.dim(0), p.dim(1), p.dim(2), p.dim(3)}).astype(f16);
    auto gb = fl::detail::pool2dBackward(tgy, b, p, 2, 2, 2, 2, 0, 0, fl::PoolingMode::AVG_INCLUDE_PADDING, pp);
    auto bn = fl::detail::batchnormBackward(gb, sm, sv, c, tg, {2}, true, 1e-5f, nullptr);
    auto gc = std::get<0>(bn);
    out(std::get<1>(bn), ggamma);
    out(std::get<2>(bn), gbeta);
    out(fl::detail::conv2dBackwardData(gc, tx, tw, 1, 1, pad, pad, 1, 1, 1, nullptr, pc)
            .astype(fl::dtype::f32),
        gx);
    out(fl::detail::conv2dBackwardFilterBias(
            gc, tx, tw, fl::Tensor(), 1, 1, pad, pad, 1, 1, 1, nullptr, nullptr, pc)
            .first.astype(fl::dtype::f32),
        gw);
  });
}

// ---- run-time kernel-mode selection (DynamicBenchmark) ----
using Bench = std::shared_ptr<fl::DynamicBenchmark>;
void* flb200_fl_benchmark_new(void) {
  try {
    fl::Tensor t({2}, fl::dtype::f32);
    auto b = t.backend().getExtension<fl::AutogradExtension>().createBenchmarkOptions();
    return b ? new Bench(b) : nullptr;
  } catch (const std::exception& e) {
    g_error = e.what();
    return nullptr;
  }
}
void flb200_fl_benchmark_free(void* h) {
  delete static_cast<Bench*>(h);
}
void flb200_fl_benchmark_mode(int on) {
  fl::DynamicBenchmark::setBenchmarkMode(on != 0);
}
// index of the option the next audited call will use, and whether tuning has finished
int flb200_fl_benchmark_state(void* h, int* complete) {
  auto opts = (*static_cast<Bench*>(h))
                  ->getOptions<fl::DynamicBenchmarkOptions<fl::B200AutogradExtension::KernelMode>>();
  if (complete) {
    *complete = opts->timingsComplete() ? 1 : 0;
  }
  return static_cast<int>(opts->currentOption());
}

int flb200_fl_conv2d_backward_tuned(
    const float* gy, const float* x, const float* w, float* gx, float* gw, int W, int H, int C,
    int N, int kW, int kH, int Cout, int Wo, int Ho, int sx, int sy, int px, int py, int dx,
    int dy, int groups, void* data_bench, void* filter_bench) {
  return guarded([&] {
    Bench db = data_bench ? *static_cast<Bench*>(data_bench) : nullptr;
    Bench fb = filter_bench ? *static_cast<Bench*>(filter_bench) : nullptr;
    auto tgy = in(gy, {Wo, Ho, Cout, N});
    auto tx = in(x, {W, H, C, N});
    auto tw = in(w, {kW, kH, C / groups, Cout});
    out(fl::detail::conv2dBackwardData(tgy, tx, tw, sx, sy, px, py, dx, dy, groups, db, nullptr),
        gx);
    out(fl::detail::conv2dBackwardFilterBias(
            tgy, tx, tw, fl::Tensor(), sx, sy, px, py, dx, dy, groups, fb, nullptr, nullptr)
            .first,
        gw);
  });
}

// ---- fl::distributed through fl::Tensor objects (f32 host buffers in, reduced values out) ----
int flb200_fl_distributed_init(const char* path, int rank, int size, int devices_per_node) {
  return guarded([&] {
    fl::distributedInit(
        fl::DistributedInit::FILE_SYSTEM, rank, size,
        {{fl::DistributedConstants::kFilePath, path ? path : ""},
         {fl::DistributedConstants::kMaxDevicePerNode, std::to_string(devices_per_node)},
         {"RENDEZVOUS_TIMEOUT_S", "60"}});
  });
}

int flb200_fl_world_rank(void) {
  return fl::getWorldRank();
}
int flb200_fl_world_size(void) {
  return fl::getWorldSize();
}

int flb200_fl_all_reduce(float* data, long long n, int async) {
  return guarded([&] {
    auto t = in(data, {static_cast<fl::Dim>(n)});
    fl::allReduce(t, async != 0);
    if (async) {
      fl::syncDistributed();
    }
    out(t, data);
  });
}

int flb200_fl_all_reduce_multiple(
    float* const* data, const long long* counts, int n, int async, int contiguous) {
  return guarded([&] {
    std::vector<fl::Tensor> held;
    held.reserve(n);
    for (int i = 0; i < n; ++i) {
      held.push_back(in(data[i], {static_cast<fl::Dim>(counts[i])}));
    }
    std::vector<fl::Tensor*> ptrs;
    for (auto& t : held) {
      ptrs.push_back(&t);
    }
    fl::allReduceMultiple(ptrs, async != 0, contiguous != 0);
    fl::syncDistributed();
    for (int i = 0; i < n; ++i) {
      out(held[i], data[i]);
    }
  });
}

} // extern "C"
