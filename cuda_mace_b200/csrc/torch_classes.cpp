// TorchScript custom classes with the names, namespaces and forward() argument lists of cuda-mace
// (cuda_mace/src/*.cpp), implemented on top of the C-ABI of libcuda_mace_b200.so:
//
//   inv_message_passing.InvariantMessagePassingTP   (src/invariant_message_passing.cpp:62-90)
//   symm_contract.SymmetricContraction              (src/symmetric_contraction.cpp:124-158)
//   linear_wmma.Linear, linear_wmma.ElementalLinear  (src/linear.cpp:105-138)
//   spherical_harmonics.SphericalHarmonics           (src/spherical_harmonics.cpp:52-69)
//   cubic_spline.CubicSpline                         (src/cubic_spline.cpp:54-68)
//
// After torch.classes.load_library(<this library>), cuda_mace/ops/*.py and models/InvariantMACE.py find the
// handles they ask for with torch.classes.<ns>.<Class>().  This file owns what the C-ABI leaves to its caller:
// output and scratch allocation through the caching allocator, argument checks, the autograd Functions
// (gradients for the float inputs only, as in the reference) and the current CUDA stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <nvtx3/nvToolsExt.h>

#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/cuda_mace_b200.h"

using torch::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

namespace {

// NVTX range around every autograd forward / backward, named after the operator (the reference pushes a range
// "cuda_mace" with a colour per operator, include/utils.h:9-21): filters for ncu / nsys, no cost when no tool listens.
struct Range {
  explicit Range(const char *name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
};

void check(int rc, const char *what) { TORCH_CHECK(rc == 0, what, " failed (", rc, "): ", cmace_last_error()); }

cmace_stream_t stream_of(const Tensor &t) {
  return (cmace_stream_t)c10::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

void check_cuda(const Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (there is no CPU implementation)");
}

bool is_f64(const Tensor &t) {
  TORCH_CHECK(t.scalar_type() == torch::kFloat32 || t.scalar_type() == torch::kFloat64, "float32 or float64 expected");
  return t.scalar_type() == torch::kFloat64;
}

Tensor int32_contig(const Tensor &t) { return t.to(torch::kInt32).contiguous(); }

std::mutex &status_mutex() {
  static std::mutex m;
  return m;
}
std::map<int, Tensor> &status_map() {
  static std::map<int, Tensor> per_device;
  return per_device;
}

// int32[1] per device that kernels with bounded waits set when a wait gives up
Tensor status_tensor(const Tensor &like) {
  std::lock_guard<std::mutex> lock(status_mutex());
  const int dev = like.device().index();
  auto &per_device = status_map();
  auto it = per_device.find(dev);
  if (it == per_device.end())
    it = per_device.emplace(dev, torch::zeros({1}, torch::dtype(torch::kInt32).device(like.device()))).first;
  return it->second;
}

Tensor status_peek(int dev) {
  std::lock_guard<std::mutex> lock(status_mutex());
  auto it = status_map().find(dev);
  return it == status_map().end() ? Tensor() : it->second;
}

// ---- edge topology: receiver CSR and, for the backward, the sender-grouped edge order --------------------
struct Topology {
  Tensor sender, receiver, row_ptr, perm, send_ptr;
  int64_t nnodes = 0, nsenders = 0, nedges = 0;
};

Topology make_topology(const Tensor &sender_list, const Tensor &receiver_list, int64_t nnodes, int64_t nsenders) {
  Topology t;
  t.sender = int32_contig(sender_list);
  t.receiver = int32_contig(receiver_list);
  t.nnodes = nnodes;
  t.nsenders = nsenders;
  t.nedges = t.sender.numel();
  t.row_ptr = torch::empty({nnodes + 1}, t.sender.options());
  check(cmace_receiver_csr(t.receiver.data_ptr<int32_t>(), t.nedges, nnodes, t.row_ptr.data_ptr<int32_t>(),
                           stream_of(t.sender)),
        "cmace_receiver_csr");
  return t;
}

void add_sender_order(Topology &t) {
  const int64_t nbytes = cmace_sender_order_workspace_bytes(t.nedges);
  Tensor ws = torch::empty({std::max<int64_t>(nbytes, 1)}, t.sender.options().dtype(torch::kUInt8));
  t.perm = torch::empty({std::max<int64_t>(t.nedges, 1)}, t.sender.options());
  t.send_ptr = torch::empty({t.nsenders + 1}, t.sender.options());
  check(cmace_sender_order(t.sender.data_ptr<int32_t>(), t.nedges, t.nsenders, t.perm.data_ptr<int32_t>(),
                           t.send_ptr.data_ptr<int32_t>(), ws.data_ptr(), nbytes, stream_of(t.sender)),
        "cmace_sender_order");
}

// ---- invariant message passing ------------------------------------------------------------------------
class IMPAutograd : public torch::autograd::Function<IMPAutograd> {
 public:
  static Tensor forward(AutogradContext *ctx, Tensor X, Tensor Y, Tensor radial, Tensor sender_list,
                        Tensor receiver_list, int64_t nnodes) {
    Range nvtx("cuda_mace_b200::message_passing::forward");
    check_cuda(X, "X");
    c10::cuda::CUDAGuard guard(X.device());
    X = X.contiguous();
    Y = Y.contiguous();
    radial = radial.contiguous();
    const int64_t C = X.size(1), E = sender_list.numel();
    TORCH_CHECK(X.dim() == 2 && Y.dim() == 2 && Y.size(0) == 16 && Y.size(1) == E, "Y must be [16, nedges]");
    TORCH_CHECK(radial.numel() == E * 4 * C, "radial must be [nedges, 4, nchannels]");
    TORCH_CHECK(Y.scalar_type() == X.scalar_type() && radial.scalar_type() == X.scalar_type(), "dtype mismatch");
    Topology topo = make_topology(sender_list, receiver_list, nnodes, X.size(0));
    Tensor out = torch::empty({nnodes, 16, C}, X.options());
    if (is_f64(X))
      check(cmace_imp_fwd_f64(X.data_ptr<double>(), Y.data_ptr<double>(), radial.data_ptr<double>(),
                              topo.sender.data_ptr<int32_t>(), topo.row_ptr.data_ptr<int32_t>(), nnodes, E, (int)C,
                              out.data_ptr<double>(), stream_of(X)),
            "cmace_imp_fwd_f64");
    else
      check(cmace_imp_fwd_f32(X.data_ptr<float>(), Y.data_ptr<float>(), radial.data_ptr<float>(),
                              topo.sender.data_ptr<int32_t>(), topo.row_ptr.data_ptr<int32_t>(), nnodes, E, (int)C,
                              out.data_ptr<float>(), stream_of(X)),
            "cmace_imp_fwd_f32");
    ctx->save_for_backward({X, Y, radial, topo.sender, topo.row_ptr});
    ctx->saved_data["nnodes"] = nnodes;
    return out;
  }

  static variable_list backward(AutogradContext *ctx, variable_list grads) {
    Range nvtx("cuda_mace_b200::message_passing::backward");
    auto saved = ctx->get_saved_variables();
    Tensor X = saved[0], Y = saved[1], radial = saved[2];
    Topology topo;
    topo.sender = saved[3];
    topo.row_ptr = saved[4];
    topo.nnodes = ctx->saved_data["nnodes"].toInt();
    topo.nsenders = X.size(0);
    topo.nedges = topo.sender.numel();
    c10::cuda::CUDAGuard guard(X.device());
    Tensor G = grads[0].contiguous();
    const int64_t C = X.size(1), E = topo.nedges;
    const bool f64 = is_f64(X);
    Tensor gradR = torch::empty_like(radial), gradY = torch::empty_like(Y);
    Tensor T = torch::empty({std::max<int64_t>(E, 1), C}, X.options());
    const int64_t nscratch = cmace_imp_bwd_scratch_elems(E, (int)C, f64 ? 1 : 0);
    Tensor scratch = torch::empty({std::max<int64_t>(nscratch, 1)}, X.options());
    add_sender_order(topo);
    Tensor gradX = torch::empty_like(X);
    if (f64) {
      check(cmace_imp_bwd_edge_f64(X.data_ptr<double>(), Y.data_ptr<double>(), radial.data_ptr<double>(),
                                   G.data_ptr<double>(), topo.sender.data_ptr<int32_t>(),
                                   topo.row_ptr.data_ptr<int32_t>(), topo.nnodes, E, (int)C, gradR.data_ptr<double>(),
                                   gradY.data_ptr<double>(), T.data_ptr<double>(),
                                   nscratch > 0 ? scratch.data_ptr<double>() : nullptr, stream_of(X)),
            "cmace_imp_bwd_edge_f64");
      check(cmace_imp_bwd_node_f64(T.data_ptr<double>(), topo.perm.data_ptr<int32_t>(),
                                   topo.send_ptr.data_ptr<int32_t>(), topo.nsenders, (int)C, gradX.data_ptr<double>(),
                                   stream_of(X)),
            "cmace_imp_bwd_node_f64");
    } else {
      check(cmace_imp_bwd_edge_f32(X.data_ptr<float>(), Y.data_ptr<float>(), radial.data_ptr<float>(),
                                   G.data_ptr<float>(), topo.sender.data_ptr<int32_t>(),
                                   topo.row_ptr.data_ptr<int32_t>(), topo.nnodes, E, (int)C, gradR.data_ptr<float>(),
                                   gradY.data_ptr<float>(), T.data_ptr<float>(),
                                   nscratch > 0 ? scratch.data_ptr<float>() : nullptr, stream_of(X)),
            "cmace_imp_bwd_edge_f32");
      check(cmace_imp_bwd_node_f32(T.data_ptr<float>(), topo.perm.data_ptr<int32_t>(),
                                   topo.send_ptr.data_ptr<int32_t>(), topo.nsenders, (int)C, gradX.data_ptr<float>(),
                                   stream_of(X)),
            "cmace_imp_bwd_node_f32");
    }
    return {gradX, gradY, gradR, Tensor(), Tensor(), Tensor()};
  }
};

// ---- Linear / ElementalLinear --------------------------------------------------------------------------
// packed tensor-core image of a float32 weight (transposed copy).  An entry keeps the source tensor alive, so its
// storage cannot be handed to another tensor of the same shape while the entry lives; the version counter catches
// in-place edits.
struct PackedEntry {
  Tensor source, packed;
};

Tensor packed_weights(const Tensor &Bt) {
  static std::mutex m;
  using Key = std::tuple<void *, int64_t, int, std::vector<int64_t>>;
  static std::map<Key, PackedEntry> cache;
  const Key key = std::make_tuple(Bt.data_ptr(), (int64_t)Bt._version(), (int)Bt.device().index(), Bt.sizes().vec());
  std::lock_guard<std::mutex> lock(m);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second.packed;
  if (cache.size() > 64) cache.clear();
  Tensor B3 = Bt.reshape({-1, Bt.size(-2), Bt.size(-1)}).contiguous();
  const int nmat = (int)B3.size(0), N = (int)B3.size(1), K = (int)B3.size(2);
  Tensor packed = torch::empty({cmace_gemm_packed_floats(nmat, N, K)}, B3.options());
  check(cmace_gemm_pack_weights_f32(B3.data_ptr<float>(), nmat, N, K, packed.data_ptr<float>(), stream_of(B3)),
        "cmace_gemm_pack_weights_f32");
  cache.emplace(key, PackedEntry{Bt, packed});
  return packed;
}

// Element grouping of a one-hot node attribute matrix [nnodes, Z], cached per tensor (it is the same tensor for every
// layer and every step of a model): node_order [nnodes] (empty when the nodes are already stored grouped by element,
// which lets the float32 kernel move whole-node boxes by TMA) and elem_start [Z + 1].  The first call for a tensor
// reads one flag back from the device; the entry keeps the source alive like the weight cache does.
struct GroupEntry {
  Tensor source, order, start;
};

GroupEntry element_grouping(const Tensor &one_hot) {
  static std::mutex m;
  using Key = std::tuple<void *, int64_t, int, std::vector<int64_t>>;
  static std::map<Key, GroupEntry> cache;
  const Key key = std::make_tuple(one_hot.data_ptr(), (int64_t)one_hot._version(), (int)one_hot.device().index(),
                                  one_hot.sizes().vec());
  std::lock_guard<std::mutex> lock(m);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 16) cache.clear();
  const int64_t N = one_hot.size(0), Z = one_hot.size(1);
  Tensor elem = one_hot.argmax(1).to(torch::kInt32).contiguous();
  const int64_t nbytes = cmace_sender_order_workspace_bytes(N);
  Tensor ws = torch::empty({std::max<int64_t>(nbytes, 1)}, elem.options().dtype(torch::kUInt8));
  Tensor order = torch::empty({std::max<int64_t>(N, 1)}, elem.options());
  Tensor start = torch::empty({Z + 1}, elem.options());
  check(cmace_group_by_element(elem.data_ptr<int32_t>(), N, (int)Z, order.data_ptr<int32_t>(),
                               start.data_ptr<int32_t>(), ws.data_ptr(), nbytes, stream_of(elem)),
        "cmace_group_by_element");
  if (N > 1 && elem.slice(0, 1, N).ge(elem.slice(0, 0, N - 1)).all().item<bool>())
    order = torch::empty({0}, elem.options());
  GroupEntry e{one_hot, order, start};
  cache.emplace(key, e);
  return e;
}

// out = scale * X @ W[z, l] per row; Wt is the transposed copy of W
Tensor linear_call(const Tensor &Xin, const Tensor &W, const Tensor &Wt, const Tensor &node_order,
                   const Tensor &elem_start, int64_t nelements, double scale) {
  Tensor X = Xin.contiguous();
  TORCH_CHECK(X.dim() == 3 && X.size(1) == 16, "X must be [nnodes, 16, K]");
  const int64_t N = X.size(0), K = X.size(2), Nout = W.size(-1);
  TORCH_CHECK(W.size(-2) == K && W.numel() == nelements * 4 * K * Nout, "weight shape does not match X");
  TORCH_CHECK(W.scalar_type() == X.scalar_type(), "X and W must have the same dtype");
  Tensor out = torch::empty({N, 16, Nout}, X.options());
  // an empty tensor stands for "no element grouping" (autograd cannot carry undefined tensors as inputs)
  const int32_t *order = node_order.defined() && node_order.numel() > 0 ? node_order.data_ptr<int32_t>() : nullptr;
  const int32_t *start = elem_start.defined() && elem_start.numel() > 0 ? elem_start.data_ptr<int32_t>() : nullptr;
  if (is_f64(X)) {
    Tensor Wc = W.contiguous();
    check(cmace_linear_f64(X.data_ptr<double>(), Wc.data_ptr<double>(), order, start, (int)nelements, N, (int)K,
                           (int)Nout, scale, out.data_ptr<double>(), stream_of(X)),
          "cmace_linear_f64");
  } else if (K % 8 == 0 && Nout % 4 == 0 && Nout <= 128) {
    Tensor packed = packed_weights(Wt);
    check(cmace_linear_tc_f32(X.data_ptr<float>(), packed.data_ptr<float>(), order, start, (int)nelements, N, (int)K,
                              (int)Nout, scale, out.data_ptr<float>(), status_tensor(X).data_ptr<int32_t>(),
                              stream_of(X)),
          "cmace_linear_tc_f32");
  } else {
    Tensor Wc = W.contiguous();
    check(cmace_linear_f32(X.data_ptr<float>(), Wc.data_ptr<float>(), order, start, (int)nelements, N, (int)K,
                           (int)Nout, scale, out.data_ptr<float>(), stream_of(X)),
          "cmace_linear_f32");
  }
  return out;
}

class LinearAutograd : public torch::autograd::Function<LinearAutograd> {
 public:
  static Tensor forward(AutogradContext *ctx, Tensor X, Tensor W, Tensor W_T, Tensor node_order, Tensor elem_start,
                        int64_t nelements) {
    Range nvtx("cuda_mace_b200::linear::forward");
    check_cuda(X, "X");
    c10::cuda::CUDAGuard guard(X.device());
    const double scale = 1.0 / std::sqrt((double)X.size(2));  // the path weight of linear_impl.cu:33
    ctx->save_for_backward({W, W_T, node_order, elem_start});
    ctx->saved_data["nelements"] = nelements;
    ctx->saved_data["scale"] = scale;
    return linear_call(X, W, W_T, node_order, elem_start, nelements, scale);
  }
  static variable_list backward(AutogradContext *ctx, variable_list grads) {
    Range nvtx("cuda_mace_b200::linear::backward");
    auto saved = ctx->get_saved_variables();
    c10::cuda::CUDAGuard guard(grads[0].device());
    Tensor dX = linear_call(grads[0], saved[1], saved[0], saved[2], saved[3], ctx->saved_data["nelements"].toInt(),
                            ctx->saved_data["scale"].toDouble());
    return {dX, Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

// ---- symmetric contraction -----------------------------------------------------------------------------
struct PlanHolder {
  cmace_symcon_plan *plan = nullptr;
  std::vector<Tensor> tables;  // the tensors the plan was made from: kept so that their addresses stay theirs
  ~PlanHolder() {
    if (plan) cmace_symcon_plan_destroy(plan);
  }
};

// The caller has made X's device current: the plan's tables are allocated on the current device.
std::shared_ptr<PlanHolder> plan_for(int64_t u3_max, const Tensor &U3_num, const Tensor &U3_idx, const Tensor &U3_val,
                                     const Tensor &U2_num, const Tensor &U2_idx, const Tensor &U2_val, int64_t w3,
                                     int64_t w2, int64_t w1, int device) {
  static std::mutex m;
  using Key = std::tuple<void *, void *, void *, void *, void *, void *, int64_t, int64_t, int64_t, int64_t, int,
                         int64_t>;
  static std::map<Key, std::shared_ptr<PlanHolder>> cache;
  const int64_t versions = (int64_t)U3_idx._version() + (int64_t)U3_val._version() + (int64_t)U2_idx._version() +
                           (int64_t)U2_val._version() + (int64_t)U3_num._version() + (int64_t)U2_num._version();
  const Key key = std::make_tuple(U3_num.data_ptr(), U3_idx.data_ptr(), U3_val.data_ptr(), U2_num.data_ptr(),
                                  U2_idx.data_ptr(), U2_val.data_ptr(), u3_max, w3, w2, w1, device, versions);
  std::lock_guard<std::mutex> lock(m);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  // host copies of the sparse tables (once per table set)
  Tensor n3 = U3_num.detach().to(torch::kCPU, torch::kInt16).contiguous();
  Tensor i3 = U3_idx.detach().to(torch::kCPU, torch::kInt32).contiguous();
  Tensor v3 = U3_val.detach().to(torch::kCPU, torch::kFloat64).contiguous();
  Tensor n2 = U2_num.detach().to(torch::kCPU, torch::kInt16).contiguous();
  Tensor i2 = U2_idx.detach().to(torch::kCPU, torch::kInt16).contiguous();
  Tensor v2 = U2_val.detach().to(torch::kCPU, torch::kFloat64).contiguous();
  auto holder = std::make_shared<PlanHolder>();
  holder->tables = {U3_num, U3_idx, U3_val, U2_num, U2_idx, U2_val};
  check(cmace_symcon_plan_create((int)u3_max, n3.data_ptr<int16_t>(), i3.data_ptr<int32_t>(), v3.data_ptr<double>(),
                                 n2.data_ptr<int16_t>(), i2.data_ptr<int16_t>(), v2.data_ptr<double>(), (int)w3,
                                 (int)w2, (int)w1, &holder->plan),
        "cmace_symcon_plan_create");
  if (cache.size() > 8) cache.clear();
  cache.emplace(key, holder);
  return holder;
}

struct PlanBox : torch::CustomClassHolder {
  std::shared_ptr<PlanHolder> holder;
};

class SymConAutograd : public torch::autograd::Function<SymConAutograd> {
 public:
  static Tensor forward(AutogradContext *ctx, Tensor X, Tensor atom_types, Tensor W3, Tensor W2, Tensor W1,
                        c10::intrusive_ptr<PlanBox> box) {
    Range nvtx("cuda_mace_b200::symmetric_contraction::forward");
    c10::cuda::CUDAGuard guard(X.device());
    X = X.contiguous();
    const int64_t N = X.size(0), C = X.size(2), Z = W3.size(0);
    Tensor out = torch::empty({N, 1, C}, X.options());
    const cmace_symcon_plan *plan = box->holder->plan;
    if (is_f64(X))
      check(cmace_symcon_fwd_f64(plan, X.data_ptr<double>(), atom_types.data_ptr<int32_t>(), W3.data_ptr<double>(),
                                 W2.data_ptr<double>(), W1.data_ptr<double>(), (int)Z, N, (int)C,
                                 out.data_ptr<double>(), stream_of(X)),
            "cmace_symcon_fwd_f64");
    else
      check(cmace_symcon_fwd_f32(plan, X.data_ptr<float>(), atom_types.data_ptr<int32_t>(), W3.data_ptr<float>(),
                                 W2.data_ptr<float>(), W1.data_ptr<float>(), (int)Z, N, (int)C, out.data_ptr<float>(),
                                 stream_of(X)),
            "cmace_symcon_fwd_f32");
    ctx->save_for_backward({X, atom_types, W3, W2, W1});
    ctx->saved_data["plan"] = box;
    return out;
  }
  static variable_list backward(AutogradContext *ctx, variable_list grads) {
    Range nvtx("cuda_mace_b200::symmetric_contraction::backward");
    auto s = ctx->get_saved_variables();
    Tensor X = s[0], atom_types = s[1], W3 = s[2], W2 = s[3], W1 = s[4];
    c10::cuda::CUDAGuard guard(X.device());
    auto box = ctx->saved_data["plan"].toCustomClass<PlanBox>();
    Tensor G = grads[0].contiguous();
    const int64_t N = X.size(0), C = X.size(2), Z = W3.size(0);
    Tensor gradX = torch::empty_like(X);
    const cmace_symcon_plan *plan = box->holder->plan;
    if (is_f64(X))
      check(cmace_symcon_bwd_f64(plan, X.data_ptr<double>(), atom_types.data_ptr<int32_t>(), W3.data_ptr<double>(),
                                 W2.data_ptr<double>(), W1.data_ptr<double>(), G.data_ptr<double>(), (int)Z, N, (int)C,
                                 gradX.data_ptr<double>(), stream_of(X)),
            "cmace_symcon_bwd_f64");
    else
      check(cmace_symcon_bwd_f32(plan, X.data_ptr<float>(), atom_types.data_ptr<int32_t>(), W3.data_ptr<float>(),
                                 W2.data_ptr<float>(), W1.data_ptr<float>(), G.data_ptr<float>(), (int)Z, N, (int)C,
                                 gradX.data_ptr<float>(), stream_of(X)),
            "cmace_symcon_bwd_f32");
    return {gradX, Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

// ---- spherical harmonics, cubic spline ------------------------------------------------------------------
class SphAutograd : public torch::autograd::Function<SphAutograd> {
 public:
  static Tensor forward(AutogradContext *ctx, Tensor xyz) {
    Range nvtx("cuda_mace_b200::spherical_harmonics::forward");
    check_cuda(xyz, "xyz");
    c10::cuda::CUDAGuard guard(xyz.device());
    xyz = xyz.contiguous();
    TORCH_CHECK(xyz.dim() == 2 && xyz.size(1) == 3, "xyz must be [nedges, 3]");
    const int64_t E = xyz.size(0);
    Tensor Y = torch::empty({16, E}, xyz.options());
    if (is_f64(xyz))
      check(cmace_sph_fwd_f64(xyz.data_ptr<double>(), E, Y.data_ptr<double>(), stream_of(xyz)), "cmace_sph_fwd_f64");
    else
      check(cmace_sph_fwd_f32(xyz.data_ptr<float>(), E, Y.data_ptr<float>(), stream_of(xyz)), "cmace_sph_fwd_f32");
    ctx->save_for_backward({xyz});
    return Y;
  }
  static variable_list backward(AutogradContext *ctx, variable_list grads) {
    Range nvtx("cuda_mace_b200::spherical_harmonics::backward");
    Tensor xyz = ctx->get_saved_variables()[0];
    c10::cuda::CUDAGuard guard(xyz.device());
    Tensor gY = grads[0].contiguous();
    Tensor gxyz = torch::empty_like(xyz);
    if (is_f64(xyz))
      check(cmace_sph_bwd_f64(xyz.data_ptr<double>(), gY.data_ptr<double>(), xyz.size(0), gxyz.data_ptr<double>(),
                              stream_of(xyz)),
            "cmace_sph_bwd_f64");
    else
      check(cmace_sph_bwd_f32(xyz.data_ptr<float>(), gY.data_ptr<float>(), xyz.size(0), gxyz.data_ptr<float>(),
                              stream_of(xyz)),
            "cmace_sph_bwd_f32");
    return {gxyz};
  }
};

class SplineAutograd : public torch::autograd::Function<SplineAutograd> {
 public:
  static Tensor forward(AutogradContext *ctx, Tensor r, Tensor r_knots, Tensor coeffs, double r_width, double r_max) {
    Range nvtx("cuda_mace_b200::cubic_spline::forward");
    check_cuda(r, "r");
    c10::cuda::CUDAGuard guard(r.device());
    r = r.contiguous();
    r_knots = r_knots.contiguous();
    coeffs = coeffs.contiguous();
    TORCH_CHECK(coeffs.dim() == 3 && coeffs.size(1) == 4, "coeffs must be [nintervals, 4, noutputs]");
    const int64_t E = r.numel(), nint = coeffs.size(0), nout = coeffs.size(2);
    Tensor R = torch::empty({E, nout}, r.options());
    if (is_f64(r))
      check(cmace_spline_fwd_f64(r.data_ptr<double>(), r_knots.data_ptr<double>(), coeffs.data_ptr<double>(), E,
                                 (int)nint, (int)nout, r_width, r_max, R.data_ptr<double>(), stream_of(r)),
            "cmace_spline_fwd_f64");
    else
      check(cmace_spline_fwd_f32(r.data_ptr<float>(), r_knots.data_ptr<float>(), coeffs.data_ptr<float>(), E, (int)nint,
                                 (int)nout, r_width, r_max, R.data_ptr<float>(), stream_of(r)),
            "cmace_spline_fwd_f32");
    ctx->save_for_backward({r, r_knots, coeffs});
    ctx->saved_data["r_width"] = r_width;
    ctx->saved_data["r_max"] = r_max;
    return R;
  }
  static variable_list backward(AutogradContext *ctx, variable_list grads) {
    Range nvtx("cuda_mace_b200::cubic_spline::backward");
    auto s = ctx->get_saved_variables();
    Tensor r = s[0], r_knots = s[1], coeffs = s[2];
    c10::cuda::CUDAGuard guard(r.device());
    Tensor gR = grads[0].contiguous();
    const int64_t E = r.numel(), nint = coeffs.size(0), nout = coeffs.size(2);
    const double r_width = ctx->saved_data["r_width"].toDouble(), r_max = ctx->saved_data["r_max"].toDouble();
    Tensor gr = torch::empty_like(r);
    if (is_f64(r))
      check(cmace_spline_bwd_f64(r.data_ptr<double>(), r_knots.data_ptr<double>(), coeffs.data_ptr<double>(),
                                 gR.data_ptr<double>(), E, (int)nint, (int)nout, r_width, r_max, gr.data_ptr<double>(),
                                 stream_of(r)),
            "cmace_spline_bwd_f64");
    else
      check(cmace_spline_bwd_f32(r.data_ptr<float>(), r_knots.data_ptr<float>(), coeffs.data_ptr<float>(),
                                 gR.data_ptr<float>(), E, (int)nint, (int)nout, r_width, r_max, gr.data_ptr<float>(),
                                 stream_of(r)),
            "cmace_spline_bwd_f32");
    return {gr, Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

}  // namespace

// ---- the classes the reference's Python layer instantiates -------------------------------------------------
class InvariantMessagePassingTP : public torch::CustomClassHolder {
 public:
  Tensor forward(Tensor X, Tensor Y, Tensor radial, Tensor sender_list, Tensor receiver_list, int64_t nnodes) {
    check_cuda(X, "X");
    c10::cuda::CUDAGuard guard(X.device());
    return IMPAutograd::apply(X, Y, radial, sender_list, receiver_list, nnodes);
  }
  std::vector<Tensor> __getstate__() { return {}; }
  void __setstate__(const std::vector<Tensor> &) {}
};

class SymmetricContraction : public torch::CustomClassHolder {
 public:
  Tensor forward(Tensor X, Tensor atom_types, int64_t U3_max_nonsparse, Tensor U3_num_nonzero, Tensor U3_indices,
                 Tensor U3_values, Tensor U2_num_nonzero, Tensor U2_indices, Tensor U2_values, Tensor U1_num_nonzero,
                 Tensor U1_index, Tensor W3, Tensor W2, Tensor W1, int64_t W3_size, int64_t W2_size, int64_t W1_size) {
    check_cuda(X, "X");
    c10::cuda::CUDAGuard guard(X.device());
    (void)U1_num_nonzero;  // accepted for signature compatibility; the reference kernel does not read them either
    (void)U1_index;        // (symmetric_contraction_impl.cu:115-117)
    auto box = c10::make_intrusive<PlanBox>();
    box->holder = plan_for(U3_max_nonsparse, U3_num_nonzero, U3_indices, U3_values, U2_num_nonzero, U2_indices,
                           U2_values, W3_size, W2_size, W1_size, (int)X.device().index());
    // the reference's buffers are [nlout, Z, w, C]; output irrep 0 is the one it contracts (impl.cu:64-76)
    auto first = [](const Tensor &w) { return (w.dim() == 4 ? w.select(0, 0) : w).contiguous(); };
    Tensor w3 = first(W3), w2 = first(W2), w1 = first(W1);
    TORCH_CHECK(w3.scalar_type() == X.scalar_type(), "X and the weights must have the same dtype");
    TORCH_CHECK(w3.size(1) == W3_size && w2.size(1) == W2_size && w1.size(1) == W1_size,
                "weight buffers do not match W3_size / W2_size / W1_size");
    return SymConAutograd::apply(X, int32_contig(atom_types), w3, w2, w1, box);
  }
  std::vector<Tensor> __getstate__() { return {}; }
  void __setstate__(const std::vector<Tensor> &) {}
};

class Linear : public torch::CustomClassHolder {
 public:
  Tensor forward(Tensor X, Tensor W, Tensor W_T) {
    check_cuda(X, "X");
    c10::cuda::CUDAGuard guard(X.device());
    Tensor none = torch::empty({0}, torch::dtype(torch::kInt32).device(X.device()));
    return LinearAutograd::apply(X, W, W_T, none, none, 1);
  }
  std::vector<Tensor> __getstate__() { return {}; }
  void __setstate__(const std::vector<Tensor> &) {}
};

class ElementalLinear : public torch::CustomClassHolder {
 public:
  // W [Z, 4, K, N], W_T [Z, 4, N, K], one_hot_encoding [nnodes, Z] (float, as in the reference)
  Tensor forward(Tensor X, Tensor W, Tensor W_T, Tensor one_hot_encoding) {
    check_cuda(X, "X");
    c10::cuda::CUDAGuard guard(X.device());
    const int64_t Z = one_hot_encoding.size(1), N = one_hot_encoding.size(0);
    TORCH_CHECK(N == X.size(0) && W.dim() == 4 && W.size(0) == Z, "one_hot_encoding must be [nnodes, Z] with W [Z, 4, K, N]");
    if (Z == 1) {  // a single-species model: every row uses W[0], no grouping needed
      Tensor none = torch::empty({0}, torch::dtype(torch::kInt32).device(X.device()));
      return LinearAutograd::apply(X, W, W_T, none, none, 1);
    }
    const GroupEntry grouping = element_grouping(one_hot_encoding);
    return LinearAutograd::apply(X, W, W_T, grouping.order, grouping.start, Z);
  }
  std::vector<Tensor> __getstate__() { return {}; }
  void __setstate__(const std::vector<Tensor> &) {}
};

class SphericalHarmonics : public torch::CustomClassHolder {
 public:
  Tensor forward(Tensor xyz) {
    check_cuda(xyz, "xyz");
    c10::cuda::CUDAGuard guard(xyz.device());
    return SphAutograd::apply(xyz);
  }
  std::vector<Tensor> __getstate__() { return {}; }
  void __setstate__(const std::vector<Tensor> &) {}
};

class CubicSpline : public torch::CustomClassHolder {
 public:
  Tensor forward(Tensor r, Tensor r_knots, Tensor coeffs, double r_width, double r_max) {
    check_cuda(r, "r");
    c10::cuda::CUDAGuard guard(r.device());
    return SplineAutograd::apply(r, r_knots, coeffs, r_width, r_max);
  }
  std::vector<Tensor> __getstate__() { return {}; }
  void __setstate__(const std::vector<Tensor> &) {}
};

// Argument names are the reference's (src/invariant_message_passing.cpp:78 - "raidal" is its spelling -,
// src/linear.cpp:110,:126, src/symmetric_contraction.cpp:129-146), so keyword calls written against it work here;
// SphericalHarmonics and CubicSpline are registered without names there too (src/spherical_harmonics.cpp:57,
// src/cubic_spline.cpp:58).
#define CMACE_PICKLE(CLS)                                                                                         \
  def_pickle([](const c10::intrusive_ptr<CLS> &self) -> std::vector<Tensor> { return self->__getstate__(); },     \
             [](const std::vector<Tensor> &state) -> c10::intrusive_ptr<CLS> {                                    \
               auto obj = c10::make_intrusive<CLS>();                                                             \
               obj->__setstate__(state);                                                                          \
               return obj;                                                                                        \
             })

TORCH_LIBRARY(inv_message_passing, m) {
  m.class_<InvariantMessagePassingTP>("InvariantMessagePassingTP")
      .def(torch::init<>(), "", {})
      .def("forward", &InvariantMessagePassingTP::forward, "",
           {torch::arg("X"), torch::arg("Y"), torch::arg("raidal"), torch::arg("sender_list"),
            torch::arg("receiver_list"), torch::arg("nnodes")})
      .CMACE_PICKLE(InvariantMessagePassingTP);
}

TORCH_LIBRARY(symm_contract, m) {
  m.class_<SymmetricContraction>("SymmetricContraction")
      .def(torch::init<>(), "", {})
      .def("forward", &SymmetricContraction::forward, "",
           {torch::arg("X"), torch::arg("atom_types"), torch::arg("U3_max_nonsparse"), torch::arg("U3_num_nonzero"),
            torch::arg("U3_indices"), torch::arg("U3_values"), torch::arg("U2_num_nonzero"), torch::arg("U2_indices"),
            torch::arg("U2_values"), torch::arg("U1_num_nonzero"), torch::arg("U1_index"), torch::arg("W3"),
            torch::arg("W2"), torch::arg("W1"), torch::arg("W3_size"), torch::arg("W2_size"), torch::arg("W1_size")})
      .CMACE_PICKLE(SymmetricContraction);
}

TORCH_LIBRARY(spherical_harmonics, m) {
  m.class_<SphericalHarmonics>("SphericalHarmonics")
      .def(torch::init<>())
      .def("forward", &SphericalHarmonics::forward)
      .CMACE_PICKLE(SphericalHarmonics);
}

TORCH_LIBRARY(cubic_spline, m) {
  m.class_<CubicSpline>("CubicSpline")
      .def(torch::init<>(), "", {})
      .def("forward", &CubicSpline::forward)
      .CMACE_PICKLE(CubicSpline);
}

TORCH_LIBRARY(linear_wmma, m) {
  m.class_<Linear>("Linear")
      .def(torch::init<>(), "", {})
      .def("forward", &Linear::forward, "", {torch::arg("X"), torch::arg("W"), torch::arg("W_T")})
      .CMACE_PICKLE(Linear);
  m.class_<ElementalLinear>("ElementalLinear")
      .def(torch::init<>(), "", {})
      .def("forward", &ElementalLinear::forward, "",
           {torch::arg("X"), torch::arg("W"), torch::arg("W_T"), torch::arg("one_hot_encoding")})
      .CMACE_PICKLE(ElementalLinear);
}

// Reads and clears what the kernels' bounded waits report (synchronises the device).  Returns 0 when every wait
// since the last call completed; otherwise a non-zero code: the outputs of the call that gave up are incomplete and
// must be discarded.  Python: torch.ops.cmace_b200_internal.check_status().
int64_t check_status_op() {
  int64_t code = cmace_imp_staged_stalled() != 0 ? 1 : 0;
  for (int dev = 0; dev < (int)c10::cuda::device_count(); ++dev) {
    Tensor t = status_peek(dev);
    if (!t.defined()) continue;
    const int64_t v = t.item<int32_t>();
    if (v != 0) {
      t.zero_();
      code = code ? code : 2 + v;
    }
  }
  return code;
}

// internal holder of a contraction plan inside an autograd node, and the status check
TORCH_LIBRARY(cmace_b200_internal, m) {
  m.class_<PlanBox>("PlanBox").def(torch::init<>());
  m.def("check_status() -> int", &check_status_op);
}
