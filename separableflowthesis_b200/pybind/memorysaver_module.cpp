// Native Python module `MemorySaver`: the five functions of the reference's pybind11 module
// (libs/MemorySaver/src/MemorySaver_cuda.cpp:105-112), same names, argument order, return order, shapes and
// dtypes, implemented as thin calls into the C ABI of libsepflow_b200.so (include/sepflow_b200.h).
//
// Built as MemorySaver.so it can take the place of the file the reference loads with
// `from ..build.lib import MemorySaver` (libs/MemorySaver/functions/MemorySaver.py:3): copy MemorySaver.so and
// libsepflow_b200.so into libs/MemorySaver/build/lib/.
//
// What the module adds over the reference's host code (MemorySaver_cuda.cpp:6-103): shape / dtype / device
// checks (the reference checks CUDA + contiguous only), a device guard, launches on torch's current stream
// instead of the legacy default stream, and the GIL released around the calls.  Outputs and the scratch
// workspace come from torch's caching allocator; the workspace is cached per (device, stream) and grown on demand.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <dlfcn.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/sepflow_b200.h"

namespace {

// ---- the C ABI, resolved at module import --------------------------------------------------------------
struct Abi {
  void* handle = nullptr;
  decltype(&sfb_workspace_bytes) workspace_bytes = nullptr;
  decltype(&sfb_max_avg_forward) max_avg_forward = nullptr;
  decltype(&sfb_max_argmax_avg_forward) max_argmax_avg_forward = nullptr;
  decltype(&sfb_max_argmax_avg_backward) max_argmax_avg_backward = nullptr;
  decltype(&sfb_compression_forward) compression_forward = nullptr;
  decltype(&sfb_compression_backward) compression_backward = nullptr;
  decltype(&sfb_last_error) last_error = nullptr;
  decltype(&sfb_status_string) status_string = nullptr;
};
Abi g_abi;

std::string module_dir() {
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&module_dir), &info) == 0 || info.dli_fname == nullptr) return ".";
  std::string path(info.dli_fname);
  const size_t slash = path.rfind('/');
  return slash == std::string::npos ? "." : path.substr(0, slash);
}

// libsepflow_b200.so is looked for in $SFB_LIB_PATH, beside this module, and where the build put it.
void load_abi() {
  std::vector<std::string> candidates;
  if (const char* env = getenv("SFB_LIB_PATH")) candidates.push_back(env);
  const std::string dir = module_dir();
  candidates.push_back(dir + "/libsepflow_b200.so");
  candidates.push_back(dir + "/../csrc/libsepflow_b200.so");
  std::string tried;
  for (const std::string& c : candidates) {
    g_abi.handle = dlopen(c.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (g_abi.handle != nullptr) break;
    tried += "\n  " + c + ": " + dlerror();
  }
  TORCH_CHECK(g_abi.handle != nullptr, "MemorySaver: libsepflow_b200.so not found (there is no fallback); tried:", tried);
#define SFB_RESOLVE(member, symbol)                                                     \
  g_abi.member = reinterpret_cast<decltype(g_abi.member)>(dlsym(g_abi.handle, symbol)); \
  TORCH_CHECK(g_abi.member != nullptr, "MemorySaver: libsepflow_b200.so lacks ", symbol)
  SFB_RESOLVE(workspace_bytes, "sfb_workspace_bytes");
  SFB_RESOLVE(max_avg_forward, "sfb_max_avg_forward");
  SFB_RESOLVE(max_argmax_avg_forward, "sfb_max_argmax_avg_forward");
  SFB_RESOLVE(max_argmax_avg_backward, "sfb_max_argmax_avg_backward");
  SFB_RESOLVE(compression_forward, "sfb_compression_forward");
  SFB_RESOLVE(compression_backward, "sfb_compression_backward");
  SFB_RESOLVE(last_error, "sfb_last_error");
  SFB_RESOLVE(status_string, "sfb_status_string");
#undef SFB_RESOLVE
}

// ---- input checks (MemorySaver_cuda.cpp:6-8, plus what the reference leaves unchecked) ------------------
void check_input(const at::Tensor& t, const char* name, at::ScalarType dtype, int64_t ndim) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", dtype, ", got ", t.scalar_type());
  TORCH_CHECK(t.dim() == ndim, name, " must have ", ndim, " dimensions, got ", t.dim());
}
void check_like(const at::Tensor& t, const char* name, at::IntArrayRef shape, at::ScalarType dtype,
                const at::Device& device) {
  check_input(t, name, dtype, static_cast<int64_t>(shape.size()));
  TORCH_CHECK(t.sizes() == shape, name, " must have shape ", shape, ", got ", t.sizes());
  TORCH_CHECK(t.device() == device, name, " is on ", t.device(), ", expected ", device);
}
sfb_shape check_pair(const at::Tensor& F1, const at::Tensor& F2) {
  check_input(F1, "img1_features_l0", at::kFloat, 4);
  check_input(F2, "img2_features_lk", at::kFloat, 4);
  TORCH_CHECK(F1.device() == F2.device(), "img1_features_l0 and img2_features_lk must be on the same device");
  TORCH_CHECK(F1.size(0) == F2.size(0) && F1.size(3) == F2.size(3), "batch / feature dimensions differ: ", F1.sizes(),
              " vs ", F2.sizes());
  sfb_shape s;
  s.B = static_cast<int32_t>(F1.size(0)); s.H1 = static_cast<int32_t>(F1.size(1)); s.W1 = static_cast<int32_t>(F1.size(2));
  s.H2 = static_cast<int32_t>(F2.size(1)); s.W2 = static_cast<int32_t>(F2.size(2)); s.C = static_cast<int32_t>(F1.size(3));
  s.Kc = 0;
  return s;
}
void check_attention(sfb_shape& s, const at::Tensor& A_u, const at::Tensor& A_v, const at::Device& dev) {
  check_input(A_u, "attention_weights_u", at::kFloat, 5);
  s.Kc = static_cast<int32_t>(A_u.size(3));
  TORCH_CHECK(s.Kc >= 1, "attention weights need at least one channel");
  check_like(A_u, "attention_weights_u", {s.B, s.H1, s.W1, s.Kc, s.W2}, at::kFloat, dev);
  check_like(A_v, "attention_weights_v", {s.B, s.H1, s.W1, s.Kc, s.H2}, at::kFloat, dev);
}

// ---- workspace cache ---------------------------------------------------------------------------------
std::mutex g_ws_mu;
std::map<std::pair<int, void*>, at::Tensor> g_ws;

at::Tensor workspace(int op, const sfb_shape& s, const at::Device& dev, cudaStream_t stream) {
  size_t bytes = g_abi.workspace_bytes(op, &s);
  if (bytes == 0) bytes = 256;  // the entry point then reports the precise reason
  std::lock_guard<std::mutex> lk(g_ws_mu);
  at::Tensor& ws = g_ws[{dev.index(), static_cast<void*>(stream)}];
  if (!ws.defined() || static_cast<size_t>(ws.numel()) < bytes)
    ws = at::empty({static_cast<int64_t>(bytes)}, at::TensorOptions().dtype(at::kByte).device(dev));
  return ws;
}

void raise_on(int rc, const char* name) {
  TORCH_CHECK(rc == SFB_OK, name, ": ", g_abi.status_string(rc), ": ", g_abi.last_error());
}

at::TensorOptions f32(const at::Tensor& like) { return like.options().dtype(at::kFloat); }
at::TensorOptions i32(const at::Tensor& like) { return like.options().dtype(at::kInt); }

// ---- the five ops --------------------------------------------------------------------------------------
// MemorySaver_cuda.cpp:10-21
std::vector<at::Tensor> max_avg_forward(at::Tensor img1_features_l0, at::Tensor img2_features_lk) {
  const at::Tensor &F1 = img1_features_l0, &F2 = img2_features_lk;
  const sfb_shape s = check_pair(F1, F2);
  const c10::cuda::CUDAGuard guard(F1.device());
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  at::Tensor MA_u = at::empty({s.B, s.H1, s.W1, 2, s.H2}, f32(F1)), MA_v = at::empty({s.B, s.H1, s.W1, 2, s.W2}, f32(F1));
  at::Tensor ws = workspace(SFB_OP_MAX_AVG_FORWARD, s, F1.device(), stream);
  int rc;
  {
    pybind11::gil_scoped_release nogil;
    rc = g_abi.max_avg_forward(F1.data_ptr<float>(), F2.data_ptr<float>(), MA_u.data_ptr<float>(), MA_v.data_ptr<float>(),
                               &s, ws.data_ptr(), static_cast<size_t>(ws.numel()), stream);
  }
  raise_on(rc, "max_avg_forward");
  return {MA_u, MA_v};
}

// MemorySaver_cuda.cpp:23-34
std::vector<at::Tensor> max_argmax_avg_forward(at::Tensor img1_features_l0, at::Tensor img2_features_lk) {
  const at::Tensor &F1 = img1_features_l0, &F2 = img2_features_lk;
  const sfb_shape s = check_pair(F1, F2);
  const c10::cuda::CUDAGuard guard(F1.device());
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  at::Tensor MA_u = at::empty({s.B, s.H1, s.W1, 2, s.H2}, f32(F1)), MA_v = at::empty({s.B, s.H1, s.W1, 2, s.W2}, f32(F1));
  at::Tensor AM_u = at::empty({s.B, s.H1, s.W1, 1, s.H2}, i32(F1)), AM_v = at::empty({s.B, s.H1, s.W1, 1, s.W2}, i32(F1));
  at::Tensor ws = workspace(SFB_OP_MAX_AVG_FORWARD, s, F1.device(), stream);
  int rc;
  {
    pybind11::gil_scoped_release nogil;
    rc = g_abi.max_argmax_avg_forward(F1.data_ptr<float>(), F2.data_ptr<float>(), MA_u.data_ptr<float>(),
                                      MA_v.data_ptr<float>(), AM_u.data_ptr<int32_t>(), AM_v.data_ptr<int32_t>(), &s,
                                      ws.data_ptr(), static_cast<size_t>(ws.numel()), stream);
  }
  raise_on(rc, "max_argmax_avg_forward");
  return {MA_u, MA_v, AM_u, AM_v};
}

// MemorySaver_cuda.cpp:55-78
std::vector<at::Tensor> max_argmax_avg_backward(at::Tensor img1_features_l0, at::Tensor img2_features_lk,
                                                at::Tensor argmax_output_u, at::Tensor argmax_output_v,
                                                at::Tensor grad_MaxAvg_u, at::Tensor grad_MaxAvg_v) {
  const at::Tensor &F1 = img1_features_l0, &F2 = img2_features_lk;
  const sfb_shape s = check_pair(F1, F2);
  const at::Device dev = F1.device();
  check_like(argmax_output_u, "argmax_output_u", {s.B, s.H1, s.W1, 1, s.H2}, at::kInt, dev);
  check_like(argmax_output_v, "argmax_output_v", {s.B, s.H1, s.W1, 1, s.W2}, at::kInt, dev);
  check_like(grad_MaxAvg_u, "grad_MaxAvg_u", {s.B, s.H1, s.W1, 2, s.H2}, at::kFloat, dev);
  check_like(grad_MaxAvg_v, "grad_MaxAvg_v", {s.B, s.H1, s.W1, 2, s.W2}, at::kFloat, dev);
  const c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  at::Tensor gF1 = at::empty_like(F1), gF2 = at::empty_like(F2);
  at::Tensor ws = workspace(SFB_OP_MAX_ARGMAX_AVG_BACKWARD, s, dev, stream);
  int rc;
  {
    pybind11::gil_scoped_release nogil;
    rc = g_abi.max_argmax_avg_backward(F1.data_ptr<float>(), F2.data_ptr<float>(), argmax_output_u.data_ptr<int32_t>(),
                                       argmax_output_v.data_ptr<int32_t>(), grad_MaxAvg_u.data_ptr<float>(),
                                       grad_MaxAvg_v.data_ptr<float>(), gF1.data_ptr<float>(), gF2.data_ptr<float>(), &s,
                                       ws.data_ptr(), static_cast<size_t>(ws.numel()), stream);
  }
  raise_on(rc, "max_argmax_avg_backward");
  return {gF1, gF2};
}

// MemorySaver_cuda.cpp:36-53 (any Kc >= 1; the reference's kernel computes two channels only,
// MemorySaver_kernel_forward.cu:20,1061)
std::vector<at::Tensor> compression_forward(at::Tensor img1_features_l0, at::Tensor img2_features_lk,
                                            at::Tensor attention_weights_u, at::Tensor attention_weights_v) {
  const at::Tensor &F1 = img1_features_l0, &F2 = img2_features_lk;
  sfb_shape s = check_pair(F1, F2);
  const at::Device dev = F1.device();
  check_attention(s, attention_weights_u, attention_weights_v, dev);
  const c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  at::Tensor C_u = at::empty({s.B, s.H1, s.W1, s.Kc, s.H2}, f32(F1)), C_v = at::empty({s.B, s.H1, s.W1, s.Kc, s.W2}, f32(F1));
  at::Tensor ws = workspace(SFB_OP_COMPRESSION_FORWARD, s, dev, stream);
  int rc;
  {
    pybind11::gil_scoped_release nogil;
    rc = g_abi.compression_forward(F1.data_ptr<float>(), F2.data_ptr<float>(), attention_weights_u.data_ptr<float>(),
                                   attention_weights_v.data_ptr<float>(), C_u.data_ptr<float>(), C_v.data_ptr<float>(), &s,
                                   ws.data_ptr(), static_cast<size_t>(ws.numel()), stream);
  }
  raise_on(rc, "compression_forward");
  return {C_u, C_v};
}

// MemorySaver_cuda.cpp:80-103
std::vector<at::Tensor> compression_backward(at::Tensor img1_features_l0, at::Tensor img2_features_lk,
                                             at::Tensor attention_weights_u, at::Tensor attention_weights_v,
                                             at::Tensor grad_compressed_output_u, at::Tensor grad_compressed_output_v) {
  const at::Tensor &F1 = img1_features_l0, &F2 = img2_features_lk;
  sfb_shape s = check_pair(F1, F2);
  const at::Device dev = F1.device();
  check_attention(s, attention_weights_u, attention_weights_v, dev);
  check_like(grad_compressed_output_u, "grad_compressed_output_u", {s.B, s.H1, s.W1, s.Kc, s.H2}, at::kFloat, dev);
  check_like(grad_compressed_output_v, "grad_compressed_output_v", {s.B, s.H1, s.W1, s.Kc, s.W2}, at::kFloat, dev);
  const c10::cuda::CUDAGuard guard(dev);
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  at::Tensor gF1 = at::empty_like(F1), gF2 = at::empty_like(F2);
  at::Tensor gA_u = at::empty_like(attention_weights_u), gA_v = at::empty_like(attention_weights_v);
  at::Tensor ws = workspace(SFB_OP_COMPRESSION_BACKWARD, s, dev, stream);
  int rc;
  {
    pybind11::gil_scoped_release nogil;
    rc = g_abi.compression_backward(F1.data_ptr<float>(), F2.data_ptr<float>(), attention_weights_u.data_ptr<float>(),
                                    attention_weights_v.data_ptr<float>(), grad_compressed_output_u.data_ptr<float>(),
                                    grad_compressed_output_v.data_ptr<float>(), gF1.data_ptr<float>(),
                                    gF2.data_ptr<float>(), gA_u.data_ptr<float>(), gA_v.data_ptr<float>(), &s,
                                    ws.data_ptr(), static_cast<size_t>(ws.numel()), stream);
  }
  raise_on(rc, "compression_backward");
  return {gF1, gF2, gA_u, gA_v};
}

}  // namespace

// Same names and doc strings as MemorySaver_cuda.cpp:105-112.
PYBIND11_MODULE(MemorySaver, m) {
  load_abi();
  m.def("max_avg_forward", &max_avg_forward, "max avg forward (CUDA)");
  m.def("max_argmax_avg_forward", &max_argmax_avg_forward, "max argmax avg forward (CUDA)");
  m.def("compression_forward", &compression_forward, "compression forward (CUDA)");
  m.def("max_argmax_avg_backward", &max_argmax_avg_backward, "max argmax avg backward (CUDA)");
  m.def("compression_backward", &compression_backward, "compression backward (CUDA)");
}
