// Host runtime: context objects, error reporting, and the CUDA-VMM symmetric allocator.
//
// Symmetric memory: every rank creates one physical allocation per buffer
// (cuMemCreate, exportable as a POSIX file descriptor), the descriptors are exchanged
// between the processes by the Python layer (SCM_RIGHTS over Unix sockets), and every
// rank maps all R allocations back to back into one reserved virtual range.  Chunk r
// then starts r*chunk_bytes after the base on every rank, which is the indexing the
// kernels and the tensor views use.  The driver API is reached through
// cudaGetDriverEntryPoint, so the library links against nothing but the static CUDA
// runtime and loads on machines without a driver.
//
// Parity: replaces the reference's NVSHMEM heap tensors (moonep_td/buffer.py:86-109);
// same role as the upstream CUDA extension's VMM + IPC mapping named in its docstring
// (moonep_td/buffer.py:1-6).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

#include "host.h"
#include "moonep.h"

namespace moonep {

static thread_local std::string g_last_error;
std::atomic<long long> g_launch_count{0};

void set_error(const std::string& s) { g_last_error = s; }

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return (int)e;
}

}  // namespace moonep

using namespace moonep;

extern "C" int moonep_version(void) { return MOONEP_VERSION; }
extern "C" const char* moonep_last_error(void) { return g_last_error.c_str(); }
extern "C" int moonep_sizeof_devctx(void) { return (int)sizeof(MoonepDevCtx); }
extern "C" long long moonep_launch_count(void) { return g_launch_count.load(); }

// ---- context ----------------------------------------------------------------------------------

enum ParamIndex {
  P_RANK = 0, P_R, P_E, P_S, P_K, P_H, P_B, P_N, P_NVS, P_EPN, P_TOKEN_PADDING, P_NUM_SMS, P_NVS_PADDED,
  P_META_STRIDE, P_WEIGHTS_OFF, P_TPE_OFF, P_PLAN_OFF, P_SRC_INFO_OFF, P_SYNC_OFF, P_R32, P_LINK_OFF, P_LOCAL_SMS,
  P_ROWFLAG_OFF, P_KP, P_TIMEOUT_MS, P_STAGE_FLAG_OFF, P_STAGE_W_OFF,
  P_PTR_STATUS, P_PTR_COUNTERS, P_PTR_ALLOC_CUM, P_PTR_EXPERT_OFF, P_PTR_TPE_PREV, P_PTR_TABLES,
  P_PTR_STATS, P_PTR_BLOCK_HIST, P_COUNT
};

extern "C" void* moonep_ctx_create(const long long* p, int nparams, const unsigned long long* hidden_peers,
                                   const unsigned long long* meta_peers, const unsigned long long* stage_peers) {
  if (nparams != P_COUNT) {
    set_error("moonep_ctx_create: expected " + std::to_string((int)P_COUNT) + " params, got " + std::to_string(nparams));
    return nullptr;
  }
  auto* h = new HostCtx();
  MoonepDevCtx& d = h->dev;
  memset(&d, 0, sizeof(d));
  d.rank = (int)p[P_RANK]; d.R = (int)p[P_R]; d.E = (int)p[P_E]; d.S = (int)p[P_S]; d.K = (int)p[P_K];
  d.H = (int)p[P_H]; d.B = (int)p[P_B]; d.N = (int)p[P_N]; d.NvS = (int)p[P_NVS]; d.epn = (int)p[P_EPN];
  d.token_padding = (int)p[P_TOKEN_PADDING]; d.num_sms = (int)p[P_NUM_SMS];
  d.nvs_padded = p[P_NVS_PADDED]; d.meta_stride = p[P_META_STRIDE];
  d.weights_off = (int)p[P_WEIGHTS_OFF]; d.tpe_off = (int)p[P_TPE_OFF]; d.plan_off = (int)p[P_PLAN_OFF];
  d.src_info_off = (int)p[P_SRC_INFO_OFF]; d.sync_off = (int)p[P_SYNC_OFF]; d.r32 = (int)p[P_R32];
  d.link_off = (int)p[P_LINK_OFF]; d.local_sms = (int)p[P_LOCAL_SMS];
  d.rowflag_off = (int)p[P_ROWFLAG_OFF]; d.kp = (int)p[P_KP];
  d.stage_flag_off = p[P_STAGE_FLAG_OFF]; d.stage_w_off = p[P_STAGE_W_OFF];
  d.timeout_ns = (unsigned long long)p[P_TIMEOUT_MS] * 1000000ull;
  d.status = (int*)p[P_PTR_STATUS]; d.counters = (int*)p[P_PTR_COUNTERS];
  d.alloc_cum = (int*)p[P_PTR_ALLOC_CUM]; d.expert_off = (int*)p[P_PTR_EXPERT_OFF];
  d.tpe_prev = (int*)p[P_PTR_TPE_PREV]; d.tables = (int*)p[P_PTR_TABLES];
  d.stats = (long long*)p[P_PTR_STATS];
  d.block_hist = (int*)p[P_PTR_BLOCK_HIST];
  if (d.R < 1 || d.R > MOONEP_MAX_RANKS || d.K < 1 || d.K > MOONEP_MAX_TOPK) {
    set_error("moonep_ctx_create: R or K out of range");
    delete h;
    return nullptr;
  }
  const size_t tbytes = sizeof(void*) * (size_t)d.R;
  void* tab = nullptr;
  if (check_cuda(cudaMalloc(&tab, 3 * tbytes), "cudaMalloc(peer tables)")) {
    delete h;
    return nullptr;
  }
  h->peer_tables = tab;
  if (check_cuda(cudaMemcpy(tab, hidden_peers, tbytes, cudaMemcpyHostToDevice), "copy hidden peers") ||
      check_cuda(cudaMemcpy((char*)tab + tbytes, meta_peers, tbytes, cudaMemcpyHostToDevice), "copy meta peers")) {
    cudaFree(tab);
    delete h;
    return nullptr;
  }
  d.hidden_peer = (uint16_t* const*)tab;
  d.meta_peer = (int* const*)((char*)tab + tbytes);
  d.stage_peer = nullptr;
  if (stage_peers != nullptr) {
    if (check_cuda(cudaMemcpy((char*)tab + 2 * tbytes, stage_peers, tbytes, cudaMemcpyHostToDevice), "copy stage peers")) {
      cudaFree(tab);
      delete h;
      return nullptr;
    }
    d.stage_peer = (unsigned char* const*)((char*)tab + 2 * tbytes);
  }
  cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, 0);
  int devid = 0;
  cudaGetDevice(&devid);
  cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, devid);
  cudaDeviceGetAttribute(&h->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, devid);
  return h;
}

extern "C" void moonep_ctx_destroy(void* ctx) {
  auto* h = (HostCtx*)ctx;
  if (!h) return;
  if (h->peer_tables) cudaFree(h->peer_tables);
  delete h;
}

extern "C" int moonep_ctx_set_pdl(void* ctx, int on) {
  auto* h = (HostCtx*)ctx;
  if (!h) return 1;
  h->enable_pdl = on ? 1 : 0;
  return 0;
}

extern "C" int moonep_ctx_set_timeout_ms(void* ctx, long long ms) {
  auto* h = (HostCtx*)ctx;
  if (!h || ms < 1) return 1;
  h->dev.timeout_ns = (unsigned long long)ms * 1000000ull;
  return 0;
}

// ---- VMM ----------------------------------------------------------------------------------------

namespace {

struct Driver {
  bool ok = false;
  std::string why;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
};

template <typename F>
bool load_sym(const char* name, F& fn, std::string& why) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    why = std::string("driver entry point not found: ") + name;
    cudaGetLastError();
    return false;
  }
  fn = (F)p;
  return true;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = load_sym("cuMemGetAllocationGranularity", d.MemGetAllocationGranularity, d.why) &&
           load_sym("cuMemCreate", d.MemCreate, d.why) &&
           load_sym("cuMemExportToShareableHandle", d.MemExportToShareableHandle, d.why) &&
           load_sym("cuMemImportFromShareableHandle", d.MemImportFromShareableHandle, d.why) &&
           load_sym("cuMemAddressReserve", d.MemAddressReserve, d.why) && load_sym("cuMemMap", d.MemMap, d.why) &&
           load_sym("cuMemSetAccess", d.MemSetAccess, d.why) && load_sym("cuMemUnmap", d.MemUnmap, d.why) &&
           load_sym("cuMemRelease", d.MemRelease, d.why) && load_sym("cuMemAddressFree", d.MemAddressFree, d.why) &&
           load_sym("cuGetErrorString", d.GetErrorString, d.why);
  });
  return d;
}

int check_cu(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return 0;
  const char* s = nullptr;
  if (driver().GetErrorString) driver().GetErrorString(r, &s);
  set_error(std::string(what) + ": CUresult " + std::to_string((int)r) + " (" + (s ? s : "?") + ")");
  return (int)r;
}

int need_driver() {
  Driver& d = driver();
  if (!d.ok) {
    set_error("CUDA driver API unavailable: " + d.why);
    return 1;
  }
  return 0;
}

CUmemAllocationProp make_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace

extern "C" int moonep_vmm_granularity(int device, unsigned long long* gran) {
  if (need_driver()) return 1;
  CUmemAllocationProp prop = make_prop(device);
  size_t g = 0;
  int rc = check_cu(driver().MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
                    "cuMemGetAllocationGranularity");
  *gran = g;
  return rc;
}

extern "C" int moonep_vmm_create(int device, unsigned long long bytes, unsigned long long* handle, int* fd) {
  if (need_driver()) return 1;
  CUmemAllocationProp prop = make_prop(device);
  CUmemGenericAllocationHandle h = 0;
  int rc = check_cu(driver().MemCreate(&h, (size_t)bytes, &prop, 0), "cuMemCreate");
  if (rc) return rc;
  int out_fd = -1;
  rc = check_cu(driver().MemExportToShareableHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                "cuMemExportToShareableHandle");
  if (rc) {
    driver().MemRelease(h);
    return rc;
  }
  *handle = (unsigned long long)h;
  *fd = out_fd;
  return 0;
}

extern "C" int moonep_vmm_import(int fd, unsigned long long* handle) {
  if (need_driver()) return 1;
  CUmemGenericAllocationHandle h = 0;
  int rc = check_cu(driver().MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                    "cuMemImportFromShareableHandle");
  *handle = (unsigned long long)h;
  return rc;
}

extern "C" int moonep_vmm_reserve(unsigned long long bytes, unsigned long long align, unsigned long long* va) {
  if (need_driver()) return 1;
  CUdeviceptr p = 0;
  int rc = check_cu(driver().MemAddressReserve(&p, (size_t)bytes, (size_t)align, 0, 0), "cuMemAddressReserve");
  *va = (unsigned long long)p;
  return rc;
}

extern "C" int moonep_vmm_map(unsigned long long va, unsigned long long bytes, unsigned long long handle, int device) {
  if (need_driver()) return 1;
  int rc = check_cu(driver().MemMap((CUdeviceptr)va, (size_t)bytes, 0, (CUmemGenericAllocationHandle)handle, 0), "cuMemMap");
  if (rc) return rc;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  rc = check_cu(driver().MemSetAccess((CUdeviceptr)va, (size_t)bytes, &acc, 1), "cuMemSetAccess");
  if (rc) driver().MemUnmap((CUdeviceptr)va, (size_t)bytes);
  return rc;
}

extern "C" int moonep_vmm_unmap(unsigned long long va, unsigned long long bytes) {
  if (need_driver()) return 1;
  return check_cu(driver().MemUnmap((CUdeviceptr)va, (size_t)bytes), "cuMemUnmap");
}

extern "C" int moonep_vmm_release(unsigned long long handle) {
  if (need_driver()) return 1;
  return check_cu(driver().MemRelease((CUmemGenericAllocationHandle)handle), "cuMemRelease");
}

extern "C" int moonep_vmm_free_va(unsigned long long va, unsigned long long bytes) {
  if (need_driver()) return 1;
  return check_cu(driver().MemAddressFree((CUdeviceptr)va, (size_t)bytes), "cuMemAddressFree");
}
