// A stand-in CUDA runtime for machines without a GPU: LD_PRELOAD it (or link it in place of libcudart) under a program
// that drives the sm_100a kernels, and every runtime call the program makes is answered on the host, checked against
// the limits of a B200, and written to a JSON-lines trace. Kernels are not executed: the point is the host side of the
// GPU path (the C++ engine, its launch geometry, tensor maps, buffer sizes, stream and event use), which a GPU-less
// build box can then test on every commit.
//
//   LD_PRELOAD=libcudart_sim.so NANOCHAT_SIM_TRACE=trace.jsonl nanochat_cli train --device cuda:0 ...
//
// What is checked (a violation is recorded in the trace and counted; with NANOCHAT_SIM_STRICT=1 the call also fails
// with cudaErrorInvalidValue, so the program under test stops where the real driver would):
//   * launches: block <= 1024 threads and within (1024, 1024, 64); grid within (2^31-1, 65535, 65535); dynamic shared
//     memory within what cudaFuncSetAttribute granted the kernel (48 KB without a grant) and within 227 KB; cluster
//     dimensions of at most 8 CTAs (16 with the non-portable attribute) that divide the grid; the kernel must have been
//     registered by its module.
//   * tensor maps (cuTensorMapEncodeTiled through cudaGetDriverEntryPoint): rank, 16-byte base alignment, strides
//     that are multiples of 16 bytes, boxes of at most 256 per dimension whose inner extent is a multiple of 16 bytes
//     and fits the swizzle span, and the whole described tensor inside one live allocation.
//   * memory: copies and memsets must stay inside live allocations; frees must name a live allocation; what is still
//     allocated at exit is listed.
//   * streams and events must be live when used.
//
// The reference ships a tool of the same kind (tools/cuda_sim/interposer.cc: an LD_PRELOAD mock of cudart / cuBLAS
// that records JSON lines and validates launch limits). This one knows the Blackwell limits and the TMA descriptor
// rules, and has no cuBLAS part because nothing here calls cuBLAS.
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <cxxabi.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

constexpr size_t kSmemOptIn = 232448;      // 227 KB: the most dynamic shared memory one CTA can be granted
constexpr size_t kSmemDefault = 49152;     // what a kernel may use without cudaFuncSetAttribute
constexpr int kSmCount = 148;

struct Kernel {
  std::string name;
  size_t smem_grant = kSmemDefault;
  bool nonportable_cluster = false;
  long long launches = 0;
};

struct State {
  std::mutex mu;
  FILE* trace = nullptr;
  bool strict = false;
  long long violations = 0, launches = 0, calls = 0, maps = 0;
  std::map<uintptr_t, size_t> allocs;                 // device allocations (host memory underneath)
  std::unordered_map<const void*, Kernel> kernels;    // host stub -> kernel
  std::unordered_map<const void*, void*> symbols;     // host shadow of a __device__ variable -> its storage
  std::set<void*> streams, events;
  uintptr_t next_handle = 0x1000;
  int device = 0;
  struct Pending { dim3 grid, block; size_t smem; cudaStream_t stream; };
  std::vector<Pending> call_stack;
  cudaError_t last_error = cudaSuccess;

  State() {
    const char* path = std::getenv("NANOCHAT_SIM_TRACE");
    if (path != nullptr && *path) trace = std::fopen(path, "w");
    const char* s = std::getenv("NANOCHAT_SIM_STRICT");
    strict = s != nullptr && s[0] == '1';
  }
};

bool g_used = false;   // a process that never called in (a child started by the program) leaves the trace alone

State& S() {
  static State* s = new State();   // never destroyed: module destructors of the program still call in at exit
  g_used = true;
  return *s;
}

std::string Demangle(const char* name) {
  int status = 0;
  char* d = abi::__cxa_demangle(name, nullptr, nullptr, &status);
  std::string out = (status == 0 && d != nullptr) ? d : name;
  std::free(d);
  if (!out.empty() && out.back() == ')') {      // drop the parameter list: the '(' that matches the last ')'
    int depth = 0;
    for (size_t i = out.size(); i-- > 0;) {
      if (out[i] == ')') ++depth;
      else if (out[i] == '(' && --depth == 0) {
        out.resize(i);
        break;
      }
    }
  }
  if (out.rfind("void ", 0) == 0) out.erase(0, 5);
  const std::string anon = "(anonymous namespace)::";
  for (size_t at; (at = out.find(anon)) != std::string::npos;) out.erase(at, anon.size());
  return out;
}

std::string Escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') o.push_back('\\');
    o.push_back(c);
  }
  return o;
}

void Emit(State& st, const std::string& line) {
  if (st.trace != nullptr) {
    std::fputs(line.c_str(), st.trace);
    std::fputc('\n', st.trace);
    std::fflush(st.trace);
  }
}

// Records a violation; returns the error the call should give back.
cudaError_t Violation(State& st, const char* call, const std::string& what) {
  ++st.violations;
  Emit(st, std::string("{\"call\":\"violation\",\"in\":\"") + call + "\",\"what\":\"" + Escape(what) + "\"}");
  if (st.trace == nullptr) std::fprintf(stderr, "[cudart_sim] %s: %s\n", call, what.c_str());
  if (st.strict) {
    st.last_error = cudaErrorInvalidValue;
    return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

// The live allocation that holds [p, p + bytes), or end() (also for a range that leaves its allocation).
bool Inside(State& st, const void* p, size_t bytes) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  auto it = st.allocs.upper_bound(a);
  if (it == st.allocs.begin()) return false;
  --it;
  return a >= it->first && a + bytes <= it->first + it->second;
}
bool IsDevicePointer(State& st, const void* p) { return Inside(st, p, 0); }

std::string Dim(const dim3& d) {
  return "[" + std::to_string(d.x) + "," + std::to_string(d.y) + "," + std::to_string(d.z) + "]";
}

cudaError_t Launch(State& st, const void* func, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                   bool pdl, const char* call) {
  ++st.launches;
  auto it = st.kernels.find(func);
  std::string name = it != st.kernels.end() ? it->second.name : "<unregistered>";
  cudaError_t rc = cudaSuccess;
  auto bad = [&](const std::string& what) {
    const cudaError_t e = Violation(st, call, name + ": " + what);
    if (e != cudaSuccess) rc = e;
  };
  if (it == st.kernels.end()) bad("launch of a function no module registered");
  const unsigned long long threads = 1ull * block.x * block.y * block.z;
  if (threads == 0 || threads > 1024 || block.x > 1024 || block.y > 1024 || block.z > 64)
    bad("block " + Dim(block) + " outside (1024, 1024, 64) / 1024 threads");
  if (grid.x == 0 || grid.y == 0 || grid.z == 0 || grid.x > 2147483647u || grid.y > 65535u || grid.z > 65535u)
    bad("grid " + Dim(grid) + " outside (2^31-1, 65535, 65535)");
  const size_t grant = it != st.kernels.end() ? it->second.smem_grant : kSmemDefault;
  if (smem > kSmemOptIn) bad("dynamic shared memory " + std::to_string(smem) + " above 232448 bytes");
  else if (smem > grant) bad("dynamic shared memory " + std::to_string(smem) + " above the kernel's grant of " +
                             std::to_string(grant) + " (cudaFuncSetAttribute not called)");
  const unsigned csize = cluster.x * cluster.y * cluster.z;
  if (csize > 1) {
    const bool np = it != st.kernels.end() && it->second.nonportable_cluster;
    if (csize > (np ? 16u : 8u)) bad("cluster of " + std::to_string(csize) + " CTAs");
    if (grid.x % cluster.x || grid.y % cluster.y || grid.z % cluster.z)
      bad("grid " + Dim(grid) + " not a multiple of cluster " + Dim(cluster));
  }
  if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread && !st.streams.count(stream))
    bad("launch on a stream that is not live");
  if (it != st.kernels.end()) ++it->second.launches;
  Emit(st, "{\"call\":\"launch\",\"kernel\":\"" + Escape(name) + "\",\"grid\":" + Dim(grid) + ",\"block\":" + Dim(block) +
               ",\"smem\":" + std::to_string(smem) + ",\"cluster\":" + Dim(cluster) + ",\"pdl\":" + (pdl ? "1" : "0") +
               ",\"stream\":" + std::to_string(reinterpret_cast<uintptr_t>(stream)) + "}");
  return rc;
}

int ElemBytes(CUtensorMapDataType t) {
  switch (t) {
    case CU_TENSOR_MAP_DATA_TYPE_UINT8: return 1;
    case CU_TENSOR_MAP_DATA_TYPE_UINT16: case CU_TENSOR_MAP_DATA_TYPE_FLOAT16: case CU_TENSOR_MAP_DATA_TYPE_BFLOAT16: return 2;
    case CU_TENSOR_MAP_DATA_TYPE_UINT64: case CU_TENSOR_MAP_DATA_TYPE_INT64: case CU_TENSOR_MAP_DATA_TYPE_FLOAT64: return 8;
    default: return 4;
  }
}

// The driver's cuTensorMapEncodeTiled, as far as its argument rules go. The descriptor is filled with a copy of the
// arguments (no device ever decodes it).
CUresult SimTensorMapEncodeTiled(CUtensorMap* map, CUtensorMapDataType dtype, cuuint32_t rank, void* base,
                                 const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                                 const cuuint32_t* elem_strides, CUtensorMapInterleave interleave,
                                 CUtensorMapSwizzle swizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  ++st.maps;
  bool ok = true;
  auto bad = [&](const std::string& what) {
    Violation(st, "cuTensorMapEncodeTiled", what);
    ok = false;
  };
  const int eb = ElemBytes(dtype);
  if (map == nullptr || rank < 1 || rank > 5) bad("rank " + std::to_string(rank) + " outside 1..5");
  else {
    if (interleave != CU_TENSOR_MAP_INTERLEAVE_NONE && rank < 3) bad("interleaved layout needs rank >= 3");
    if (reinterpret_cast<uintptr_t>(base) % 16) bad("base address not 16-byte aligned");
    unsigned long long extent = eb;
    for (cuuint32_t i = 0; i < rank; ++i) {
      if (dims[i] == 0 || dims[i] > (1ull << 32)) bad("dimension " + std::to_string(i) + " = " + std::to_string(dims[i]));
      if (box[i] == 0 || box[i] > 256) bad("box " + std::to_string(i) + " = " + std::to_string(box[i]) + " outside 1..256");
      if (elem_strides[i] == 0 || elem_strides[i] > 8) bad("element stride " + std::to_string(i));
      if (i > 0) {
        const cuuint64_t s = strides[i - 1];
        if (s % 16 || s >= (1ull << 40)) bad("stride " + std::to_string(i) + " = " + std::to_string(s) + " bytes is not a multiple of 16");
        extent += (dims[i] - 1) * s;
      } else {
        extent += (dims[0] - 1) * static_cast<unsigned long long>(eb);
      }
    }
    const unsigned long long inner = 1ull * box[0] * eb;
    if (inner % 16) bad("inner box extent of " + std::to_string(inner) + " bytes is not a multiple of 16");
    const unsigned span = swizzle == CU_TENSOR_MAP_SWIZZLE_32B ? 32 : swizzle == CU_TENSOR_MAP_SWIZZLE_64B ? 64
                          : swizzle == CU_TENSOR_MAP_SWIZZLE_128B ? 128 : 0;
    if (span != 0 && inner > span) bad("inner box extent of " + std::to_string(inner) + " bytes exceeds the " +
                                       std::to_string(span) + "-byte swizzle span");
    if (!Inside(st, base, extent)) bad("tensor of " + std::to_string(extent) + " bytes is not inside one live allocation");
  }
  std::string d = "[", b = "[";
  for (cuuint32_t i = 0; i < rank && i < 5; ++i) {
    d += (i ? "," : "") + std::to_string(dims[i]);
    b += (i ? "," : "") + std::to_string(box[i]);
  }
  Emit(st, "{\"call\":\"tensor_map\",\"rank\":" + std::to_string(rank) + ",\"elem_bytes\":" + std::to_string(eb) +
               ",\"dims\":" + d + "],\"box\":" + b + "],\"swizzle\":" + std::to_string(static_cast<int>(swizzle)) + "}");
  if (!ok && st.strict) return CUDA_ERROR_INVALID_VALUE;
  if (map != nullptr) {
    std::memset(map, 0, sizeof(*map));
    std::memcpy(map, &base, sizeof(base));
  }
  return CUDA_SUCCESS;
}

void Report() {
  if (!g_used) return;
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  size_t live_bytes = 0;
  for (auto& a : st.allocs) live_bytes += a.second;
  std::string per = "{";
  bool first = true;
  for (auto& k : st.kernels) {
    if (k.second.launches == 0) continue;
    per += std::string(first ? "" : ",") + "\"" + Escape(k.second.name) + "\":" + std::to_string(k.second.launches);
    first = false;
  }
  per += "}";
  Emit(st, "{\"call\":\"summary\",\"launches\":" + std::to_string(st.launches) + ",\"tensor_maps\":" +
               std::to_string(st.maps) + ",\"violations\":" + std::to_string(st.violations) + ",\"live_allocations\":" +
               std::to_string(st.allocs.size()) + ",\"live_bytes\":" + std::to_string(live_bytes) +
               ",\"live_streams\":" + std::to_string(st.streams.size()) + ",\"live_events\":" +
               std::to_string(st.events.size()) + ",\"per_kernel\":" + per + "}");
}

struct AtExit {
  AtExit() { std::atexit(Report); }
} g_at_exit;

}  // namespace

extern "C" {

// ---- module registration (what nvcc's generated host code calls at load time)
void** __cudaRegisterFatBinary(void*) {
  static void* handle_storage[1];
  return handle_storage;
}
void __cudaRegisterFatBinaryEnd(void**) {}
void __cudaUnregisterFatBinary(void**) {}
void __cudaRegisterFunction(void**, const char* host_fun, char*, const char* device_name, int, uint3*, uint3*, dim3*,
                            dim3*, int*) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  st.kernels[host_fun].name = Demangle(device_name);
}
void __cudaRegisterVar(void**, char* host_var, char*, const char*, int, size_t size, int, int) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  void* p = nullptr;
  if (posix_memalign(&p, 256, size ? size : 1) != 0) return;
  std::memset(p, 0, size);
  st.symbols[host_var] = p;
  st.allocs[reinterpret_cast<uintptr_t>(p)] = size;   // a __device__ variable is device memory like any other
}
unsigned __cudaPushCallConfiguration(dim3 grid, dim3 block, size_t smem, struct CUstream_st* stream) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  st.call_stack.push_back({grid, block, smem, stream});
  return 0;
}
cudaError_t __cudaPopCallConfiguration(dim3* grid, dim3* block, size_t* smem, void* stream) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  if (st.call_stack.empty()) return cudaErrorInvalidConfiguration;
  const State::Pending p = st.call_stack.back();
  st.call_stack.pop_back();
  *grid = p.grid, *block = p.block, *smem = p.smem;
  *static_cast<cudaStream_t*>(stream) = p.stream;
  return cudaSuccess;
}

// ---- devices
cudaError_t cudaGetDeviceCount(int* n) {
  *n = 1;
  return cudaSuccess;
}
cudaError_t cudaSetDevice(int d) {
  if (d != 0) return cudaErrorInvalidDevice;
  S().device = d;
  return cudaSuccess;
}
cudaError_t cudaGetDevice(int* d) {
  *d = S().device;
  return cudaSuccess;
}
cudaError_t cudaGetDeviceProperties_v2(cudaDeviceProp* p, int d) {
  if (d != 0) return cudaErrorInvalidDevice;
  std::memset(p, 0, sizeof(*p));
  std::snprintf(p->name, sizeof(p->name), "NVIDIA B200 (simulated runtime)");
  p->major = 10, p->minor = 0;
  p->totalGlobalMem = 183359ull << 20;
  p->multiProcessorCount = kSmCount;
  p->sharedMemPerBlock = kSmemDefault;
  p->sharedMemPerBlockOptin = kSmemOptIn;
  p->sharedMemPerMultiprocessor = 233472;
  p->maxThreadsPerBlock = 1024;
  p->warpSize = 32;
  p->l2CacheSize = 126 << 20;
  return cudaSuccess;
}
cudaError_t cudaDeviceGetAttribute(int* value, cudaDeviceAttr attr, int d) {
  if (d != 0) return cudaErrorInvalidDevice;
  switch (attr) {
    case cudaDevAttrMultiProcessorCount: *value = kSmCount; break;
    case cudaDevAttrMaxSharedMemoryPerBlockOptin: *value = static_cast<int>(kSmemOptIn); break;
    case cudaDevAttrMaxSharedMemoryPerBlock: *value = static_cast<int>(kSmemDefault); break;
    case cudaDevAttrComputeCapabilityMajor: *value = 10; break;
    case cudaDevAttrComputeCapabilityMinor: *value = 0; break;
    case cudaDevAttrMaxThreadsPerBlock: *value = 1024; break;
    case cudaDevAttrWarpSize: *value = 32; break;
    case cudaDevAttrClusterLaunch: *value = 1; break;
    case cudaDevAttrL2CacheSize: *value = 126 << 20; break;
    default: *value = 0; break;
  }
  return cudaSuccess;
}
cudaError_t cudaDeviceSynchronize(void) { return cudaSuccess; }
cudaError_t cudaGetLastError(void) {
  State& st = S();
  const cudaError_t e = st.last_error;
  st.last_error = cudaSuccess;
  return e;
}
const char* cudaGetErrorString(cudaError_t e) {
  return e == cudaSuccess ? "no error" : e == cudaErrorInvalidValue ? "invalid argument (simulated runtime)"
                                                                    : "error (simulated runtime)";
}
cudaError_t cudaGetDriverEntryPoint(const char* symbol, void** fn, unsigned long long,
                                    cudaDriverEntryPointQueryResult* result) {
  if (std::strcmp(symbol, "cuTensorMapEncodeTiled") == 0) {
    *fn = reinterpret_cast<void*>(&SimTensorMapEncodeTiled);
    if (result != nullptr) *result = cudaDriverEntryPointSuccess;
    return cudaSuccess;
  }
  *fn = nullptr;
  if (result != nullptr) *result = cudaDriverEntryPointSymbolNotFound;
  return cudaErrorSymbolNotFound;
}

// ---- memory
cudaError_t cudaMalloc(void** p, size_t bytes) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  void* q = nullptr;
  if (posix_memalign(&q, 256, bytes ? bytes : 1) != 0) return cudaErrorMemoryAllocation;
  // untouched pages cost nothing, so a multi-GB activation buffer of a real configuration still fits a small host
  st.allocs[reinterpret_cast<uintptr_t>(q)] = bytes;
  *p = q;
  Emit(st, "{\"call\":\"malloc\",\"bytes\":" + std::to_string(bytes) + "}");
  return cudaSuccess;
}
cudaError_t cudaFree(void* p) {
  if (p == nullptr) return cudaSuccess;
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  auto it = st.allocs.find(reinterpret_cast<uintptr_t>(p));
  if (it == st.allocs.end()) return Violation(st, "cudaFree", "pointer is not a live allocation");
  Emit(st, "{\"call\":\"free\",\"bytes\":" + std::to_string(it->second) + "}");
  st.allocs.erase(it);
  std::free(p);
  return cudaSuccess;
}
cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t stream) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  ++st.calls;
  cudaError_t rc = cudaSuccess;
  const bool dst_dev = kind == cudaMemcpyHostToDevice || kind == cudaMemcpyDeviceToDevice ||
                       (kind == cudaMemcpyDefault && IsDevicePointer(st, dst));
  const bool src_dev = kind == cudaMemcpyDeviceToHost || kind == cudaMemcpyDeviceToDevice ||
                       (kind == cudaMemcpyDefault && IsDevicePointer(st, src));
  if (dst_dev && !Inside(st, dst, bytes))
    rc = Violation(st, "cudaMemcpyAsync", "destination of " + std::to_string(bytes) + " bytes leaves its allocation");
  if (src_dev && !Inside(st, src, bytes))
    rc = Violation(st, "cudaMemcpyAsync", "source of " + std::to_string(bytes) + " bytes leaves its allocation");
  if (stream != nullptr && !st.streams.count(stream)) rc = Violation(st, "cudaMemcpyAsync", "stream is not live");
  if (rc != cudaSuccess) return rc;
  if ((!dst_dev || Inside(st, dst, bytes)) && (!src_dev || Inside(st, src, bytes))) std::memmove(dst, src, bytes);
  Emit(st, "{\"call\":\"memcpy\",\"bytes\":" + std::to_string(bytes) + ",\"kind\":" + std::to_string(kind) + "}");
  return cudaSuccess;
}
cudaError_t cudaMemsetAsync(void* p, int value, size_t bytes, cudaStream_t stream) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  ++st.calls;
  if (!Inside(st, p, bytes))
    return Violation(st, "cudaMemsetAsync", "range of " + std::to_string(bytes) + " bytes leaves its allocation");
  if (stream != nullptr && !st.streams.count(stream)) return Violation(st, "cudaMemsetAsync", "stream is not live");
  std::memset(p, value, bytes);
  return cudaSuccess;
}
cudaError_t cudaMemset2DAsync(void* p, size_t pitch, int value, size_t width, size_t height, cudaStream_t stream) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  ++st.calls;
  if (height == 0 || width == 0) return cudaSuccess;
  if (width > pitch) return Violation(st, "cudaMemset2DAsync", "width above pitch");
  if (!Inside(st, p, (height - 1) * pitch + width))
    return Violation(st, "cudaMemset2DAsync", "rows leave their allocation");
  if (stream != nullptr && !st.streams.count(stream)) return Violation(st, "cudaMemset2DAsync", "stream is not live");
  for (size_t r = 0; r < height; ++r) std::memset(static_cast<char*>(p) + r * pitch, value, width);
  return cudaSuccess;
}
cudaError_t cudaGetSymbolAddress(void** p, const void* symbol) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  auto it = st.symbols.find(symbol);
  if (it == st.symbols.end()) return cudaErrorInvalidSymbol;
  *p = it->second;
  return cudaSuccess;
}

// ---- streams and events
cudaError_t cudaStreamCreateWithFlags(cudaStream_t* s, unsigned) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  void* h = reinterpret_cast<void*>(st.next_handle += 16);
  st.streams.insert(h);
  *s = static_cast<cudaStream_t>(h);
  return cudaSuccess;
}
cudaError_t cudaStreamDestroy(cudaStream_t s) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  if (!st.streams.erase(s)) return Violation(st, "cudaStreamDestroy", "stream is not live");
  return cudaSuccess;
}
cudaError_t cudaStreamSynchronize(cudaStream_t s) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  if (s != nullptr && !st.streams.count(s)) return Violation(st, "cudaStreamSynchronize", "stream is not live");
  return cudaSuccess;
}
cudaError_t cudaEventCreateWithFlags(cudaEvent_t* e, unsigned) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  void* h = reinterpret_cast<void*>(st.next_handle += 16);
  st.events.insert(h);
  *e = static_cast<cudaEvent_t>(h);
  return cudaSuccess;
}
cudaError_t cudaEventDestroy(cudaEvent_t e) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  if (!st.events.erase(e)) return Violation(st, "cudaEventDestroy", "event is not live");
  return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t e, cudaStream_t s) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  if (!st.events.count(e)) return Violation(st, "cudaEventRecord", "event is not live");
  if (s != nullptr && !st.streams.count(s)) return Violation(st, "cudaEventRecord", "stream is not live");
  return cudaSuccess;
}
cudaError_t cudaStreamWaitEvent(cudaStream_t s, cudaEvent_t e, unsigned) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  if (!st.events.count(e)) return Violation(st, "cudaStreamWaitEvent", "event is not live");
  if (s != nullptr && !st.streams.count(s)) return Violation(st, "cudaStreamWaitEvent", "stream is not live");
  return cudaSuccess;
}

// ---- kernels
cudaError_t cudaFuncSetAttribute(const void* func, cudaFuncAttribute attr, int value) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  auto it = st.kernels.find(func);
  if (it == st.kernels.end()) return Violation(st, "cudaFuncSetAttribute", "function no module registered");
  if (attr == cudaFuncAttributeMaxDynamicSharedMemorySize) {
    if (value < 0 || static_cast<size_t>(value) > kSmemOptIn)
      return Violation(st, "cudaFuncSetAttribute", it->second.name + ": " + std::to_string(value) +
                                                       " bytes of dynamic shared memory above 232448");
    it->second.smem_grant = static_cast<size_t>(value);
  } else if (attr == cudaFuncAttributeNonPortableClusterSizeAllowed) {
    it->second.nonportable_cluster = value != 0;
  }
  return cudaSuccess;
}
cudaError_t cudaLaunchKernel(const void* func, dim3 grid, dim3 block, void**, size_t smem, cudaStream_t stream) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  return Launch(st, func, grid, block, smem, stream, dim3(1, 1, 1), false, "cudaLaunchKernel");
}
cudaError_t cudaLaunchKernelExC(const cudaLaunchConfig_t* cfg, const void* func, void**) {
  State& st = S();
  std::lock_guard<std::mutex> lock(st.mu);
  dim3 cluster(1, 1, 1);
  bool pdl = false;
  for (unsigned i = 0; i < cfg->numAttrs; ++i) {
    const cudaLaunchAttribute& a = cfg->attrs[i];
    if (a.id == cudaLaunchAttributeClusterDimension)
      cluster = dim3(a.val.clusterDim.x, a.val.clusterDim.y, a.val.clusterDim.z);
    else if (a.id == cudaLaunchAttributeProgrammaticStreamSerialization)
      pdl = a.val.programmaticStreamSerializationAllowed != 0;
  }
  return Launch(st, func, cfg->gridDim, cfg->blockDim, cfg->dynamicSmemBytes, cfg->stream, cluster, pdl,
                "cudaLaunchKernelExC");
}
cudaError_t cudaOccupancyMaxActiveClusters(int* clusters, const void*, const cudaLaunchConfig_t* cfg) {
  unsigned size = 1;
  for (unsigned i = 0; i < cfg->numAttrs; ++i)
    if (cfg->attrs[i].id == cudaLaunchAttributeClusterDimension)
      size = cfg->attrs[i].val.clusterDim.x * cfg->attrs[i].val.clusterDim.y * cfg->attrs[i].val.clusterDim.z;
  *clusters = kSmCount / (size ? size : 1);
  return cudaSuccess;
}

}  // extern "C"
