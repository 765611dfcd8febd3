// Symmetric memory runtime: one cudaMalloc'd heap per rank, shared with the other ranks of the
// node through CUDA IPC handles, plus the communicator object that launches the collective kernels
// of comm_kernels.cu over it.  Handle exchange itself happens in Python over torch.distributed.
#include "symm.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <cstring>
#include <vector>

#include "himuon.h"

namespace py = pybind11;

namespace himuon {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("himuon symm: ") + what + ": " + cudaGetErrorString(e));
}

static py::tuple symm_alloc(int64_t nbytes) {
  void* p = nullptr;
  check(cudaMalloc(&p, static_cast<size_t>(nbytes)), "cudaMalloc");
  check(cudaMemset(p, 0, static_cast<size_t>(nbytes)), "cudaMemset");
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  return py::make_tuple(reinterpret_cast<int64_t>(p), py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
}

static int64_t symm_open(const py::bytes& handle) {
  std::string s = handle;
  if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("himuon symm: malformed IPC handle");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, s.data(), sizeof(h));
  void* p = nullptr;
  check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<int64_t>(p);
}

static void symm_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }
static void symm_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }

// A tensor over raw device memory that this module does not own (heap slices, peer mappings).
static at::Tensor tensor_view(int64_t ptr, std::vector<int64_t> shape, const std::string& dtype, int64_t device) {
  at::ScalarType st = dtype == "bf16" ? at::kBFloat16 : dtype == "f32" ? at::kFloat : dtype == "i32" ? at::kInt
                    : dtype == "u8" ? at::kByte : at::kLong;
  const c10::Device dev(at::kCUDA, static_cast<c10::DeviceIndex>(device));
  auto opts = at::TensorOptions().dtype(st).device(dev);
  // The target device is stated, not inferred from the pointer: a peer's memory mapped through the virtual-memory
  // API reports the peer as its device, while every kernel that touches the view runs on this rank's device.
  return at::from_blob(reinterpret_cast<void*>(ptr), shape, [](void*) {}, opts, dev);
}

class Comm {
 public:
  // mc_ptr: multicast address of the heap (0 when the heap is not bound to a multicast object)
  Comm(int rank, int world, std::vector<int64_t> heap_ptrs, double timeout_s, int64_t mc_ptr)
      : heaps_(std::move(heap_ptrs)), mc_(reinterpret_cast<char*>(mc_ptr)) {
    if (world < 1 || world > kMaxSrc || static_cast<int>(heaps_.size()) != world)
      throw std::runtime_error("himuon symm: world size must be 1..8 with one heap pointer per rank");
    peers_.world = world;
    peers_.rank = rank;
    for (int r = 0; r < kMaxSrc; ++r) peers_.flags[r] = r < world ? reinterpret_cast<int*>(heaps_[r]) : nullptr;
    set_timeout(timeout_s);
    peers_.status = status_word_ptr();
    check(cudaMalloc(&epoch_, 2 * kCommMaxBlocks * sizeof(int)), "cudaMalloc(epoch)");
    check(cudaMemset(epoch_, 0, 2 * kCommMaxBlocks * sizeof(int)), "cudaMemset(epoch)");
  }
  ~Comm() {
    if (epoch_) cudaFree(epoch_);
  }
  void set_timeout(double s) { peers_.limit_ns = static_cast<unsigned long long>(s * 1e9); }
  int64_t peer_ptr(int r) const { return heaps_.at(r); }
  static int64_t flag_bytes() { return kCommFlagBytes; }

  void barrier(int channel) { peer_barrier(peers_, epoch_, at::cuda::getCurrentCUDAStream().stream(), channel); }

  // In-place all-reduce of the same heap region on every rank.
  void allreduce(int64_t offset_bytes, int64_t n_elems, bool fp32, double scale, int64_t max_blocks, int64_t algo) {
    if (peers_.world == 1) return;
    TORCH_CHECK(offset_bytes % 16 == 0, "himuon allreduce: the region must start on a 16-byte boundary");
    if (algo == 3) {                                   // through the NVLink switch (multimem)
      TORCH_CHECK(mc_ != nullptr, "himuon allreduce: this heap has no multicast mapping");
      allreduce_nvls(peers_, mc_ + offset_bytes, n_elems, fp32 ? 1 : 0, static_cast<float>(scale), epoch_,
                     static_cast<int>(max_blocks), at::cuda::getCurrentCUDAStream().stream());
      return;
    }
    CommBufs b{};
    for (int r = 0; r < peers_.world; ++r) b.ptr[r] = reinterpret_cast<char*>(heaps_[r]) + offset_bytes;
    allreduce_symm(peers_, b, n_elems, fp32 ? 1 : 0, static_cast<float>(scale), epoch_, static_cast<int>(max_blocks),
                   at::cuda::getCurrentCUDAStream().stream(), static_cast<int>(algo));
  }
  // out = beta * out + scale * sum over ranks of the heap region at offset_bytes (out.numel() elements of out's dtype).
  void reduce_to(int64_t offset_bytes, at::Tensor out, double scale, double beta, bool multicast) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous(), "himuon reduce_to: contiguous CUDA output expected");
    TORCH_CHECK(offset_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0,
                "himuon reduce_to: 16-byte aligned regions expected");
    if (multicast && peers_.world > 1) {
      TORCH_CHECK(mc_ != nullptr, "himuon reduce_to: this heap has no multicast mapping");
      reduce_nvls(mc_ + offset_bytes, out.data_ptr(), out.numel(), out.scalar_type() == at::kFloat ? 1 : 0,
                  static_cast<float>(scale), static_cast<float>(beta), at::cuda::getCurrentCUDAStream().stream());
      return;
    }
    CommBufs b{};
    for (int r = 0; r < peers_.world; ++r) b.ptr[r] = reinterpret_cast<char*>(heaps_[r]) + offset_bytes;
    reduce_replicas(b, peers_.world, out.data_ptr(), out.numel(), out.scalar_type() == at::kFloat ? 1 : 0,
                    static_cast<float>(scale), at::cuda::getCurrentCUDAStream().stream(), static_cast<float>(beta));
  }
  void copy_segments(const at::Tensor& segs, int64_t n_segs, int64_t total_units, int64_t max_blocks) {
    TORCH_CHECK(segs.is_cuda() && segs.numel() >= n_segs * (int64_t)sizeof(CopySeg), "himuon copy_segments: table too small");
    multi_copy(reinterpret_cast<const CopySeg*>(segs.data_ptr()), static_cast<int>(n_segs), total_units,
               static_cast<int>(max_blocks), at::cuda::getCurrentCUDAStream().stream());
  }

 private:
  std::vector<int64_t> heaps_;
  char* mc_ = nullptr;
  CommPeers peers_{};
  int* epoch_ = nullptr;
};

void bind_vmm(py::module_& m);

void bind_symm(py::module_& m) {
  bind_vmm(m);
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_open", &symm_open);
  m.def("symm_close", &symm_close);
  m.def("symm_free", &symm_free);
  m.def("tensor_view", &tensor_view);
  m.def("multi_copy_units", [](int64_t bytes) { return multi_copy_units(bytes); });
  py::class_<Comm>(m, "Comm")
      .def(py::init<int, int, std::vector<int64_t>, double, int64_t>(), py::arg("rank"), py::arg("world"), py::arg("heap_ptrs"),
           py::arg("timeout_s"), py::arg("mc_ptr") = 0)
      .def("set_timeout", &Comm::set_timeout)
      .def("peer_ptr", &Comm::peer_ptr)
      .def_static("flag_bytes", &Comm::flag_bytes)
      .def("barrier", &Comm::barrier, py::arg("channel") = 0)
      .def("allreduce", &Comm::allreduce, py::arg("offset_bytes"), py::arg("n_elems"), py::arg("fp32"), py::arg("scale"),
           py::arg("max_blocks") = 0, py::arg("algo") = 0)
      .def("reduce_to", &Comm::reduce_to, py::arg("offset_bytes"), py::arg("out"), py::arg("scale"), py::arg("beta") = 0.0,
           py::arg("multicast") = false)
      .def("copy_segments", &Comm::copy_segments);
}

}  // namespace himuon
