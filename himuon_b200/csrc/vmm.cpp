// Symmetric memory on the CUDA virtual-memory API, with an NVLink-switch multicast mapping (NVLS).
//
// The default heap of symm.cpp is a cudaMalloc'd block shared through CUDA IPC handles; that is all the peer-load /
// peer-store kernels need.  The `multimem` instructions (switch-side reduction and broadcast) need more: every rank's
// physical memory must be bound to one multicast object, which only works for memory created with cuMemCreate.  This
// file provides that second kind of heap:
//
//   vmm_alloc          cuMemCreate + map + export as a POSIX file descriptor
//   vmm_import         duplicate a peer's descriptor (pidfd_getfd), import it and map it here
//   mc_create/import   the multicast object: created by rank 0, imported by the others
//   mc_add_device      every rank adds its device ...
//   mc_bind            ... then binds its own physical memory at offset 0 ...
//   mc_map             ... and maps the multicast object: loads/stores through this address go to all ranks
//   vmm_release_all    unbind, unmap and release everything, multicast first
//
// The driver entry points are fetched through the runtime (no link against libcuda), so the library still loads on a
// machine without a driver.  Handle exchange between the ranks (pid, fd numbers) happens in Python over
// torch.distributed.  The reference has no counterpart (it reaches NVLS only through NCCL).
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace himuon {

namespace {

template <typename Fn>
Fn driver_fn(const char* name, int version = 12010) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  const cudaError_t e = cudaGetDriverEntryPointByVersion(name, &p, version, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
    throw std::runtime_error(std::string("himuon vmm: driver entry point ") + name + " is not available");
  return reinterpret_cast<Fn>(p);
}

void ck(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string("himuon vmm: ") + what + " failed with CUresult " + std::to_string(static_cast<int>(r)));
}

struct Driver {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*McCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*McAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*McBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*McUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*McGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
};

const Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.MemCreate = driver_fn<decltype(d.MemCreate)>("cuMemCreate");
    d.MemRelease = driver_fn<decltype(d.MemRelease)>("cuMemRelease");
    d.MemAddressReserve = driver_fn<decltype(d.MemAddressReserve)>("cuMemAddressReserve");
    d.MemAddressFree = driver_fn<decltype(d.MemAddressFree)>("cuMemAddressFree");
    d.MemMap = driver_fn<decltype(d.MemMap)>("cuMemMap");
    d.MemUnmap = driver_fn<decltype(d.MemUnmap)>("cuMemUnmap");
    d.MemSetAccess = driver_fn<decltype(d.MemSetAccess)>("cuMemSetAccess");
    d.MemExport = driver_fn<decltype(d.MemExport)>("cuMemExportToShareableHandle");
    d.MemImport = driver_fn<decltype(d.MemImport)>("cuMemImportFromShareableHandle");
    d.MemGranularity = driver_fn<decltype(d.MemGranularity)>("cuMemGetAllocationGranularity");
    d.McCreate = driver_fn<decltype(d.McCreate)>("cuMulticastCreate");
    d.McAddDevice = driver_fn<decltype(d.McAddDevice)>("cuMulticastAddDevice");
    d.McBindMem = driver_fn<decltype(d.McBindMem)>("cuMulticastBindMem");
    d.McUnbind = driver_fn<decltype(d.McUnbind)>("cuMulticastUnbind");
    d.McGranularity = driver_fn<decltype(d.McGranularity)>("cuMulticastGetGranularity");
    d.DeviceGetAttribute = driver_fn<decltype(d.DeviceGetAttribute)>("cuDeviceGetAttribute");
  });
  return d;
}

CUmemAllocationProp mem_prop(int device) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

CUmulticastObjectProp mc_prop(int n_devices, size_t size) {
  CUmulticastObjectProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.numDevices = static_cast<unsigned>(n_devices);
  prop.size = size;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

// Everything this process created, so that teardown can run in the one safe order.
struct Mapping { CUdeviceptr va; size_t size; CUmemGenericAllocationHandle handle; };
struct Registry {
  std::mutex mu;
  std::vector<Mapping> own, peers;
  struct Mc { CUmemGenericAllocationHandle handle; size_t size; CUdeviceptr va; int device; bool bound; };
  std::vector<Mc> mcs;
  std::vector<int> fds;
};
Registry& reg() {
  static Registry r;
  return r;
}

CUdeviceptr map_handle(CUmemGenericAllocationHandle h, size_t size, size_t gran, int device) {
  const Driver& d = drv();
  CUdeviceptr va = 0;
  ck(d.MemAddressReserve(&va, size, gran, 0, 0), "cuMemAddressReserve");
  ck(d.MemMap(va, size, 0, h, 0), "cuMemMap");
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  ck(d.MemSetAccess(va, size, &acc, 1), "cuMemSetAccess");
  return va;
}

// A descriptor of another process of this user, duplicated into this one (Linux >= 5.6).
int dup_remote_fd(int pid, int remote_fd) {
  if (pid == static_cast<int>(getpid())) return dup(remote_fd);
  const int pidfd = static_cast<int>(syscall(SYS_pidfd_open, pid, 0));
  if (pidfd < 0) throw std::runtime_error(std::string("himuon vmm: pidfd_open: ") + std::strerror(errno));
  const int fd = static_cast<int>(syscall(SYS_pidfd_getfd, pidfd, remote_fd, 0));
  const int err = errno;
  close(pidfd);
  if (fd < 0) throw std::runtime_error(std::string("himuon vmm: pidfd_getfd: ") + std::strerror(err));
  return fd;
}

}  // namespace

// 1 when the device can take part in an NVLink multicast object.
static bool vmm_multicast_supported(int device) {
  try {
    int v = 0;
    if (drv().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return false;
    return v != 0;
  } catch (const std::exception&) {
    return false;
  }
}

// Allocation size (bytes) that both cuMemCreate and a multicast object of `n_devices` accept for `nbytes`.
static int64_t vmm_round_size(int64_t nbytes, int device, int n_devices) {
  const Driver& d = drv();
  size_t g = 0, gm = 0;
  const CUmemAllocationProp prop = mem_prop(device);
  ck(d.MemGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (n_devices > 1 && vmm_multicast_supported(device)) {
    const CUmulticastObjectProp mp = mc_prop(n_devices, static_cast<size_t>(nbytes));
    if (d.McGranularity(&gm, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) gm = 0;
  }
  if (gm > g) g = gm;
  return static_cast<int64_t>((static_cast<size_t>(nbytes) + g - 1) / g * g);
}

// -> (index of the allocation, mapped address, exported descriptor)
static py::tuple vmm_alloc(int64_t nbytes, int device) {
  const Driver& d = drv();
  const CUmemAllocationProp prop = mem_prop(device);
  CUmemGenericAllocationHandle h;
  ck(d.MemCreate(&h, static_cast<size_t>(nbytes), &prop, 0), "cuMemCreate");
  size_t g = 0;
  ck(d.MemGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  const CUdeviceptr va = map_handle(h, static_cast<size_t>(nbytes), g, device);
  if (cudaMemset(reinterpret_cast<void*>(va), 0, static_cast<size_t>(nbytes)) != cudaSuccess)
    throw std::runtime_error("himuon vmm: cudaMemset of the new heap failed");
  int fd = -1;
  ck(d.MemExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  r.own.push_back({va, static_cast<size_t>(nbytes), h});
  r.fds.push_back(fd);
  return py::make_tuple(static_cast<int64_t>(r.own.size() - 1), static_cast<int64_t>(va), fd);
}

// Maps a peer's allocation (its pid and descriptor number as exchanged by the ranks) into this process.
static int64_t vmm_import(int pid, int remote_fd, int64_t nbytes, int device) {
  const Driver& d = drv();
  const int fd = dup_remote_fd(pid, remote_fd);
  CUmemGenericAllocationHandle h;
  const CUresult res = d.MemImport(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  ck(res, "cuMemImportFromShareableHandle");
  const CUmemAllocationProp prop = mem_prop(device);
  size_t g = 0;
  ck(d.MemGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  const CUdeviceptr va = map_handle(h, static_cast<size_t>(nbytes), g, device);
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  r.peers.push_back({va, static_cast<size_t>(nbytes), h});
  return static_cast<int64_t>(va);
}

// Rank 0: -> (index of the multicast object, exported descriptor)
static py::tuple mc_create(int n_devices, int64_t nbytes, int device) {
  const Driver& d = drv();
  const CUmulticastObjectProp prop = mc_prop(n_devices, static_cast<size_t>(nbytes));
  CUmemGenericAllocationHandle h;
  ck(d.McCreate(&h, &prop), "cuMulticastCreate");
  int fd = -1;
  ck(d.MemExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle(multicast)");
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  r.mcs.push_back({h, static_cast<size_t>(nbytes), 0, device, false});
  r.fds.push_back(fd);
  return py::make_tuple(static_cast<int64_t>(r.mcs.size() - 1), fd);
}

static int64_t mc_import(int pid, int remote_fd, int64_t nbytes, int device) {
  const Driver& d = drv();
  const int fd = dup_remote_fd(pid, remote_fd);
  CUmemGenericAllocationHandle h;
  const CUresult res = d.MemImport(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  ck(res, "cuMemImportFromShareableHandle(multicast)");
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  r.mcs.push_back({h, static_cast<size_t>(nbytes), 0, device, false});
  return static_cast<int64_t>(r.mcs.size() - 1);
}

static void mc_add_device(int64_t mc, int device) {
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  ck(drv().McAddDevice(r.mcs.at(mc).handle, device), "cuMulticastAddDevice");
}

// Binds allocation `alloc` (index from vmm_alloc) at offset 0 of the multicast object.  Call after every rank has
// added its device.
static void mc_bind(int64_t mc, int64_t alloc) {
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  Registry::Mc& m = r.mcs.at(mc);
  const Mapping& a = r.own.at(alloc);
  if (a.size != m.size) throw std::runtime_error("himuon vmm: multicast object and allocation differ in size");
  ck(drv().McBindMem(m.handle, 0, a.handle, 0, a.size, 0), "cuMulticastBindMem");
  m.bound = true;
}

// Maps the multicast object; call after every rank has bound its memory.
static int64_t mc_map(int64_t mc) {
  const Driver& d = drv();
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  Registry::Mc& m = r.mcs.at(mc);
  size_t g = 0;
  const CUmulticastObjectProp prop = mc_prop(2, m.size);
  if (d.McGranularity(&g, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) g = 2u << 20;
  m.va = map_handle(m.handle, m.size, g, m.device);
  return static_cast<int64_t>(m.va);
}

// Teardown in the only safe order: multicast mappings and bindings first, then peer mappings, then own memory.
// Every rank must have stopped touching the heap (device idle, ranks at a barrier) before any rank calls this.
static void vmm_release_all() {
  const Driver& d = drv();
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  for (auto& m : r.mcs) {
    if (m.va) { d.MemUnmap(m.va, m.size); d.MemAddressFree(m.va, m.size); m.va = 0; }
    if (m.bound) { d.McUnbind(m.handle, m.device, 0, m.size); m.bound = false; }
    d.MemRelease(m.handle);
  }
  r.mcs.clear();
  for (auto& p : r.peers) { d.MemUnmap(p.va, p.size); d.MemAddressFree(p.va, p.size); d.MemRelease(p.handle); }
  r.peers.clear();
  for (auto& p : r.own) { d.MemUnmap(p.va, p.size); d.MemAddressFree(p.va, p.size); d.MemRelease(p.handle); }
  r.own.clear();
  for (int fd : r.fds) close(fd);
  r.fds.clear();
}

void bind_vmm(py::module_& m) {
  m.def("vmm_multicast_supported", &vmm_multicast_supported);
  m.def("vmm_round_size", &vmm_round_size);
  m.def("vmm_alloc", &vmm_alloc);
  m.def("vmm_import", &vmm_import);
  m.def("mc_create", &mc_create);
  m.def("mc_import", &mc_import);
  m.def("mc_add_device", &mc_add_device);
  m.def("mc_bind", &mc_bind);
  m.def("mc_map", &mc_map);
  m.def("vmm_release_all", &vmm_release_all);
}

}  // namespace himuon
