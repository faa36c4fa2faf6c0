// Symmetric heap for one NVLink domain.
//
// Every rank owns one region; all regions are mapped into every rank at
// `window_base + rank * bytes_per_rank`, so "the same buffer on peer r" is a fixed offset away.
// Replaces the NVSHMEM heap + peer-pointer lookup and the CUDA-IPC helper of the reference
// (odc/primitives/utils.py:54-81, csrc/tensor_ipc/tensor_ipc.cu:24-57).
//
// vmm mode: address space is reserved once; physical memory is created in growth steps with the
// CUDA virtual-memory API, exported as POSIX file descriptors, sent to the peers over unix
// datagram sockets (SCM_RIGHTS) and mapped at the same offset of the owner's window.
// ipc mode: one cudaMalloc slab per rank shared with legacy cudaIpc handles.
//
// Driver entry points are resolved at run time (no link-time dependency on libcuda), so the
// library also loads on a machine without a GPU driver.
#include "symm_heap.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <poll.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <deque>
#include <stdexcept>
#include <string>
#include <vector>

namespace odc {

namespace {

struct Driver {
  decltype(&cuMemAddressReserve) AddressReserve = nullptr;
  decltype(&cuMemAddressFree) AddressFree = nullptr;
  decltype(&cuMemCreate) Create = nullptr;
  decltype(&cuMemRelease) Release = nullptr;
  decltype(&cuMemMap) Map = nullptr;
  decltype(&cuMemUnmap) Unmap = nullptr;
  decltype(&cuMemSetAccess) SetAccess = nullptr;
  decltype(&cuMemExportToShareableHandle) Export = nullptr;
  decltype(&cuMemImportFromShareableHandle) Import = nullptr;
  decltype(&cuMemGetAllocationGranularity) Granularity = nullptr;
  decltype(&cuGetErrorString) ErrorString = nullptr;
  decltype(&cuMemGetAddressRange) AddressRange = nullptr;
};

template <typename F>
void resolve(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    throw std::runtime_error(std::string("CUDA driver entry point not available: ") + name);
  }
  *out = reinterpret_cast<F>(p);
}

Driver& drv() {
  static Driver d;
  static bool ready = false;
  if (!ready) {
    resolve("cuMemAddressReserve", &d.AddressReserve);
    resolve("cuMemAddressFree", &d.AddressFree);
    resolve("cuMemCreate", &d.Create);
    resolve("cuMemRelease", &d.Release);
    resolve("cuMemMap", &d.Map);
    resolve("cuMemUnmap", &d.Unmap);
    resolve("cuMemSetAccess", &d.SetAccess);
    resolve("cuMemExportToShareableHandle", &d.Export);
    resolve("cuMemImportFromShareableHandle", &d.Import);
    resolve("cuMemGetAllocationGranularity", &d.Granularity);
    resolve("cuGetErrorString", &d.ErrorString);
    resolve("cuMemGetAddressRange", &d.AddressRange);
    ready = true;
  }
  return d;
}

void check_cu(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) {
    const char* msg = nullptr;
    drv().ErrorString(r, &msg);
    throw std::runtime_error(std::string(what) + " failed: " + (msg ? msg : "unknown driver error"));
  }
}

void check_rt(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
  }
}

struct FdMsg {
  int src;
  unsigned long long seq;
  unsigned long long size;
  int fd;
};

sockaddr_un abstract_addr(const std::string& token, int rank, socklen_t* len) {
  sockaddr_un a;
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  std::string name = "odc_b200_" + token + "_" + std::to_string(rank);
  if (name.size() + 1 >= sizeof(a.sun_path)) throw std::runtime_error("socket name too long");
  a.sun_path[0] = '\0';  // abstract namespace: no file, vanishes with the process
  memcpy(a.sun_path + 1, name.data(), name.size());
  *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  return a;
}

}  // namespace

struct Heap {
  int rank = 0, world = 1, device = 0;
  size_t bytes_per_rank = 0;
  bool vmm = true;
  std::string token;
  CUdeviceptr window = 0;  // vmm: base of world * bytes_per_rank reservation
  std::vector<uintptr_t> bases;
  size_t mapped = 0;
  std::vector<CUmemGenericAllocationHandle> handles;  // own + imported, released at destroy
  std::vector<void*> ipc_opened;
  void* ipc_slab = nullptr;
  int sock = -1;
  unsigned long long seq = 0;
  std::deque<FdMsg> early;
  int recv_timeout_ms = 120000;
};

static void send_fd(Heap* h, int dst, int fd, unsigned long long size) {
  socklen_t alen;
  sockaddr_un addr = abstract_addr(h->token, dst, &alen);
  unsigned long long payload[3] = {static_cast<unsigned long long>(h->rank), h->seq, size};
  iovec iov{payload, sizeof(payload)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_name = &addr;
  msg.msg_namelen = alen;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (int attempt = 0; attempt < 2000; ++attempt) {
    if (sendmsg(h->sock, &msg, 0) >= 0) return;
    if (errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN || errno == ENOBUFS) {
      usleep(5000);  // peer socket not bound yet or its queue is full
      continue;
    }
    break;
  }
  throw std::runtime_error(std::string("sendmsg(fd) to rank ") + std::to_string(dst) + ": " + strerror(errno));
}

static FdMsg recv_fd(Heap* h) {
  pollfd p{h->sock, POLLIN, 0};
  int pr = poll(&p, 1, h->recv_timeout_ms);
  if (pr <= 0) throw std::runtime_error("timed out waiting for a peer's memory handle");
  unsigned long long payload[3];
  iovec iov{payload, sizeof(payload)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t n = recvmsg(h->sock, &msg, 0);
  if (n != static_cast<ssize_t>(sizeof(payload))) throw std::runtime_error("short handle message");
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_type != SCM_RIGHTS) throw std::runtime_error("handle message carried no descriptor");
  FdMsg m;
  m.src = static_cast<int>(payload[0]);
  m.seq = payload[1];
  m.size = payload[2];
  memcpy(&m.fd, CMSG_DATA(c), sizeof(int));
  return m;
}

Heap* heap_create(int rank, int world, int device, size_t bytes_per_rank, const std::string& mode,
                  const std::string& token) {
  check_rt(cudaSetDevice(device), "cudaSetDevice");
  check_rt(cudaFree(nullptr), "context creation");
  Heap* h = new Heap();
  h->rank = rank;
  h->world = world;
  h->device = device;
  h->bytes_per_rank = bytes_per_rank;
  h->vmm = (mode == "vmm");
  h->token = token;
  h->bases.assign(world, 0);
  try {
    if (h->vmm) {
      Driver& d = drv();
      CUmemAllocationProp prop;
      memset(&prop, 0, sizeof(prop));
      prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
      prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      prop.location.id = device;
      prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t gran = 0;
      check_cu(d.Granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM), "cuMemGetAllocationGranularity");
      if (bytes_per_rank % gran != 0) throw std::runtime_error("heap size is not a multiple of the granularity");
      check_cu(d.AddressReserve(&h->window, bytes_per_rank * world, gran, 0, 0), "cuMemAddressReserve");
      for (int r = 0; r < world; ++r) h->bases[r] = static_cast<uintptr_t>(h->window) + bytes_per_rank * r;
      if (world > 1) {
        h->sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
        if (h->sock < 0) throw std::runtime_error("socket() failed");
        socklen_t alen;
        sockaddr_un addr = abstract_addr(token, rank, &alen);
        if (bind(h->sock, reinterpret_cast<sockaddr*>(&addr), alen) != 0)
          throw std::runtime_error(std::string("bind() failed: ") + strerror(errno));
      }
    } else {
      check_rt(cudaMalloc(&h->ipc_slab, bytes_per_rank), "cudaMalloc(slab)");
      check_rt(cudaMemset(h->ipc_slab, 0, bytes_per_rank), "cudaMemset(slab)");
      h->bases[rank] = reinterpret_cast<uintptr_t>(h->ipc_slab);
      h->mapped = bytes_per_rank;
    }
  } catch (...) {
    heap_destroy(h);
    throw;
  }
  return h;
}

void heap_grow(Heap* h, size_t new_size) {
  if (!h->vmm) throw std::runtime_error("heap_grow applies to vmm mode only");
  if (new_size <= h->mapped) return;
  if (new_size > h->bytes_per_rank) throw std::runtime_error("heap_grow beyond the reserved window");
  Driver& d = drv();
  size_t size = new_size - h->mapped;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = h->device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = h->device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;

  CUmemGenericAllocationHandle mine;
  check_cu(d.Create(&mine, size, &prop, 0), "cuMemCreate");
  h->handles.push_back(mine);
  CUdeviceptr at = static_cast<CUdeviceptr>(h->bases[h->rank] + h->mapped);
  check_cu(d.Map(at, size, 0, mine, 0), "cuMemMap(own)");
  check_cu(d.SetAccess(at, size, &access, 1), "cuMemSetAccess(own)");
  check_rt(cudaMemset(reinterpret_cast<void*>(at), 0, size), "cudaMemset(new pages)");
  check_rt(cudaDeviceSynchronize(), "cudaDeviceSynchronize");

  if (h->world > 1) {
    int fd = -1;
    check_cu(d.Export(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
    for (int k = 1; k < h->world; ++k) send_fd(h, (h->rank + k) % h->world, fd, size);
    close(fd);
    int got = 0;
    std::vector<char> seen(h->world, 0);
    auto take = [&](const FdMsg& m) {
      if (m.src < 0 || m.src >= h->world || seen[m.src]) throw std::runtime_error("unexpected handle message");
      if (m.size != size) throw std::runtime_error("peer grew its heap by a different amount (allocation order differs)");
      CUmemGenericAllocationHandle ph;
      check_cu(d.Import(&ph, reinterpret_cast<void*>(static_cast<uintptr_t>(m.fd)),
                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle");
      close(m.fd);
      h->handles.push_back(ph);
      CUdeviceptr pat = static_cast<CUdeviceptr>(h->bases[m.src] + h->mapped);
      check_cu(d.Map(pat, size, 0, ph, 0), "cuMemMap(peer)");
      check_cu(d.SetAccess(pat, size, &access, 1), "cuMemSetAccess(peer)");
      seen[m.src] = 1;
      ++got;
    };
    for (auto it = h->early.begin(); it != h->early.end();) {
      if (it->seq == h->seq) {
        take(*it);
        it = h->early.erase(it);
      } else {
        ++it;
      }
    }
    while (got < h->world - 1) {
      FdMsg m = recv_fd(h);
      if (m.seq == h->seq) {
        take(m);
      } else {
        h->early.push_back(m);  // a faster peer is already one growth step ahead
      }
    }
  }
  h->mapped = new_size;
  h->seq += 1;
}

std::string heap_ipc_handle(Heap* h) {
  if (h->vmm) throw std::runtime_error("ipc handle requested from a vmm heap");
  cudaIpcMemHandle_t hd;
  check_rt(cudaIpcGetMemHandle(&hd, h->ipc_slab), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&hd), sizeof(hd));
}

void heap_ipc_open(Heap* h, int r, const std::string& bytes) {
  if (bytes.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad ipc handle size");
  cudaIpcMemHandle_t hd;
  memcpy(&hd, bytes.data(), sizeof(hd));
  void* p = nullptr;
  check_rt(cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  h->ipc_opened.push_back(p);
  h->bases[r] = reinterpret_cast<uintptr_t>(p);
}

uintptr_t heap_base(Heap* h, int r) { return h->bases.at(r); }
size_t heap_mapped(Heap* h) { return h->mapped; }

void heap_destroy(Heap* h) {
  if (!h) return;
  cudaDeviceSynchronize();
  if (h->vmm) {
    Driver& d = drv();
    if (h->window) {
      if (h->mapped) {
        int nwin = h->world;
        for (int r = 0; r < nwin; ++r) d.Unmap(static_cast<CUdeviceptr>(h->bases[r]), h->mapped);
      }
      for (auto hd : h->handles) d.Release(hd);
      d.AddressFree(h->window, h->bytes_per_rank * h->world);
    }
    if (h->sock >= 0) close(h->sock);
    for (auto& m : h->early) close(m.fd);
  } else {
    for (void* p : h->ipc_opened) cudaIpcCloseMemHandle(p);
    if (h->ipc_slab) cudaFree(h->ipc_slab);
  }
  delete h;
}

// Allocation-relative IPC export of an arbitrary device pointer (counterpart of the reference's
// get_ipc_handle / reconstruct_tensor, csrc/tensor_ipc/tensor_ipc.cu:24-57).  Errors are thrown,
// never exit().
std::string ipc_export(const void* ptr) {
  CUdeviceptr base = 0;
  size_t size = 0;
  check_cu(drv().AddressRange(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)), "cuMemGetAddressRange");
  cudaIpcMemHandle_t hd;
  check_rt(cudaIpcGetMemHandle(&hd, reinterpret_cast<void*>(base)), "cudaIpcGetMemHandle");
  unsigned long long off = reinterpret_cast<uintptr_t>(ptr) - static_cast<uintptr_t>(base);
  std::string out(reinterpret_cast<const char*>(&hd), sizeof(hd));
  out.append(reinterpret_cast<const char*>(&off), sizeof(off));
  return out;
}

void* ipc_import(const std::string& bytes) {
  if (bytes.size() != sizeof(cudaIpcMemHandle_t) + sizeof(unsigned long long))
    throw std::runtime_error("bad ipc blob size");
  cudaIpcMemHandle_t hd;
  unsigned long long off;
  memcpy(&hd, bytes.data(), sizeof(hd));
  memcpy(&off, bytes.data() + sizeof(hd), sizeof(off));
  void* p = nullptr;
  check_rt(cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return static_cast<char*>(p) + off;
}

}  // namespace odc
