// Device memory with generic compute-data compression for the [tokens, neurons] activation streams.
//
// The training step is bound by the bytes it moves through HBM, and most of those bytes are ReLU-sparse bf16
// activations (x, x*y, dy, dx: half or more of the entries are exactly zero). Memory created with
// CU_MEM_ALLOCATION_COMP_GENERIC is compressed losslessly by the memory system between L2 and HBM, which
// raises the effective bandwidth for such data without any change to the kernels that read and write it.
// The two functions below have the signature torch's pluggable allocator expects; Python puts them behind a
// `torch.cuda.MemPool` that only the activation buffers of the kernel path allocate from
// (utils/compressed_pool.py). Every driver entry point is resolved at run time, so the library has no link
// dependency on libcuda; nothing here outlives the process or changes a device setting.
#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/types.h>

#include <mutex>
#include <unordered_map>

#include "bdh_kernels.h"

namespace {

template <typename Fn>
Fn entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

struct Driver {
  CUresult (*getAttr)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*propFromHandle)(CUmemAllocationProp*, CUmemGenericAllocationHandle) = nullptr;
  bool ok = false;
  Driver() {
    getAttr = entry<decltype(getAttr)>("cuDeviceGetAttribute");
    granularity = entry<decltype(granularity)>("cuMemGetAllocationGranularity");
    create = entry<decltype(create)>("cuMemCreate");
    release = entry<decltype(release)>("cuMemRelease");
    reserve = entry<decltype(reserve)>("cuMemAddressReserve");
    addressFree = entry<decltype(addressFree)>("cuMemAddressFree");
    map = entry<decltype(map)>("cuMemMap");
    unmap = entry<decltype(unmap)>("cuMemUnmap");
    setAccess = entry<decltype(setAccess)>("cuMemSetAccess");
    propFromHandle = entry<decltype(propFromHandle)>("cuMemGetAllocationPropertiesFromHandle");
    ok = getAttr && granularity && create && release && reserve && addressFree && map && unmap && setAccess &&
         propFromHandle;
  }
};

Driver& drv() {
  static Driver d;
  return d;
}

struct Block {
  CUmemGenericAllocationHandle handle;
  size_t size;
  bool compressed;
};
std::mutex g_mu;
std::unordered_map<void*, Block> g_blocks;
long long g_bytes = 0, g_compressed_bytes = 0;

CUmemAllocationProp props(int device, bool compressed) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.allocFlags.compressionType = compressed ? CU_MEM_ALLOCATION_COMP_GENERIC : CU_MEM_ALLOCATION_COMP_NONE;
  return p;
}

}  // namespace

// 1 when the device offers generic compression for VMM allocations, 0 when not, -1 when the driver entry points
// could not be resolved.
extern "C" int bdh_comp_supported(int device) {
  if (!drv().ok) return -1;
  cudaFree(nullptr);                                  // a context on this thread
  int v = 0;
  if (drv().getAttr(&v, CU_DEVICE_ATTRIBUTE_GENERIC_COMPRESSION_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v ? 1 : 0;
}

// Pluggable-allocator entry points. A block that cannot be created compressible is created plain (and counted
// as such), so an allocation only fails when the device is out of memory.
extern "C" void* bdh_comp_alloc(ssize_t size, int device, cudaStream_t) {
  if (!drv().ok || size <= 0) return nullptr;
  cudaFree(nullptr);
  for (int attempt = 0; attempt < 2; ++attempt) {
    const bool compressed = attempt == 0;
    CUmemAllocationProp p = props(device, compressed);
    size_t gran = 0;
    if (drv().granularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || gran == 0) continue;
    const size_t bytes = (static_cast<size_t>(size) + gran - 1) / gran * gran;
    CUmemGenericAllocationHandle h;
    if (drv().create(&h, bytes, &p, 0) != CUDA_SUCCESS) continue;
    bool got = compressed;
    if (compressed) {
      // the driver may silently hand out plain memory: ask what the handle really is
      CUmemAllocationProp q{};
      if (drv().propFromHandle(&q, h) == CUDA_SUCCESS) got = q.allocFlags.compressionType == CU_MEM_ALLOCATION_COMP_GENERIC;
    }
    CUdeviceptr va = 0;
    if (drv().reserve(&va, bytes, gran, 0, 0) != CUDA_SUCCESS) {
      drv().release(h);
      continue;
    }
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (drv().map(va, bytes, 0, h, 0) != CUDA_SUCCESS) {
      drv().addressFree(va, bytes);
      drv().release(h);
      continue;
    }
    if (drv().setAccess(va, bytes, &acc, 1) != CUDA_SUCCESS) {
      drv().unmap(va, bytes);
      drv().addressFree(va, bytes);
      drv().release(h);
      continue;
    }
    std::lock_guard<std::mutex> lock(g_mu);
    g_blocks[reinterpret_cast<void*>(va)] = Block{h, bytes, got};
    g_bytes += static_cast<long long>(bytes);
    if (got) g_compressed_bytes += static_cast<long long>(bytes);
    return reinterpret_cast<void*>(va);
  }
  return nullptr;
}

extern "C" void bdh_comp_free(void* ptr, size_t, cudaStream_t) {
  if (!ptr || !drv().ok) return;
  Block b;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_blocks.find(ptr);
    if (it == g_blocks.end()) return;
    b = it->second;
    g_blocks.erase(it);
    g_bytes -= static_cast<long long>(b.size);
    if (b.compressed) g_compressed_bytes -= static_cast<long long>(b.size);
  }
  cudaDeviceSynchronize();                            // (segments are released rarely: when the pool is emptied)
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  drv().unmap(va, b.size);
  drv().addressFree(va, b.size);
  drv().release(b.handle);
}

// out = {bytes held, bytes of them that the driver reports as compressible}
extern "C" void bdh_comp_stats(long long* out2) {
  std::lock_guard<std::mutex> lock(g_mu);
  out2[0] = g_bytes;
  out2[1] = g_compressed_bytes;
}
