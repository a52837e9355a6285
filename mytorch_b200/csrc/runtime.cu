// Runtime part of the C ABI: error text, stream-ordered pooled allocation,
// copies, streams, events, the device status word and per-kernel-class timing.
#include "common.cuh"
#include <cstdlib>
#include "prof.cuh"
#include <nvtx3/nvToolsExt.h>
#include <stdarg.h>
#include <atomic>
#include <mutex>
#include <vector>

namespace mt {

static thread_local std::string g_err;
static std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool overlap_launches() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("MT_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

static constexpr int kMaxDev = 16;
static int* g_flag[kMaxDev] = {nullptr};
static int g_sms[kMaxDev] = {0};
static bool g_pool_ready[kMaxDev] = {false};
static std::mutex g_mu;

int* device_flag_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_flag[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_flag[dev] = p;
  }
  return g_flag[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= kMaxDev) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

// ---- timing of one kernel class --------------------------------------------
static int g_prof_kind = 0;
struct ProfRec { cudaEvent_t a, b; double flops; };
static std::vector<ProfRec> g_prof;
static std::vector<ProfRec> g_prof_free;

int prof_kind() { return g_prof_kind; }
ProfScope::ProfScope(int kind, cudaStream_t s, double flops) : active_(false), s_(s) {
  if (kind != g_prof_kind || g_prof_kind == 0) return;
  ProfRec r;
  if (!g_prof_free.empty()) { r = g_prof_free.back(); g_prof_free.pop_back(); }
  else {
    if (cudaEventCreate(&r.a) != cudaSuccess) return;
    if (cudaEventCreate(&r.b) != cudaSuccess) return;
  }
  r.flops = flops;
  cudaEventRecord(r.a, s);
  g_prof.push_back(r);
  active_ = true;
}
ProfScope::~ProfScope() {
  if (active_) cudaEventRecord(g_prof.back().b, s_);
}

}  // namespace mt

using namespace mt;

extern "C" {

const char* mt_last_error(void) { return g_err.c_str(); }
int mt_version(void) { return 100; }
int64_t mt_launch_count(void) { return g_launches.load(); }

// NVTX ranges on the calling thread. The header-only NVTX 3 binding looks for an attached tool on
// first use; without one both calls return at once, so they cost nothing outside a profiler.
int mt_range_push(const char* name) {
  MT_REQUIRE(name != nullptr, "range_push: no name");
  nvtxRangePushA(name);
  return MT_OK;
}
int mt_range_pop(void) {
  nvtxRangePop();
  return MT_OK;
}

int mt_device_count(int* count) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
  *count = n;
  return MT_OK;
}
int mt_set_device(int device) { MT_CHECK_CUDA(cudaSetDevice(device)); return MT_OK; }
int mt_get_device(int* device) { MT_CHECK_CUDA(cudaGetDevice(device)); return MT_OK; }
int mt_device_sm_count(int* count) { *count = sm_count(); return MT_OK; }

static int ensure_pool() {
  int dev = 0;
  MT_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < kMaxDev && !g_pool_ready[dev]) {
    cudaMemPool_t pool;
    MT_CHECK_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t thr = UINT64_MAX;  // keep freed blocks cached in the pool
    MT_CHECK_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thr));
    g_pool_ready[dev] = true;
  }
  return MT_OK;
}

int mt_malloc(void** ptr, size_t bytes, void* stream) {
  *ptr = nullptr;
  if (bytes == 0) bytes = 16;
  int rc = ensure_pool();
  if (rc) return rc;
  MT_CHECK_CUDA(cudaMallocAsync(ptr, bytes, as_stream(stream)));
  return MT_OK;
}
int mt_free(void* ptr, void* stream) {
  if (!ptr) return MT_OK;
  MT_CHECK_CUDA(cudaFreeAsync(ptr, as_stream(stream)));
  return MT_OK;
}
int mt_host_alloc(void** ptr, size_t bytes) { MT_CHECK_CUDA(cudaMallocHost(ptr, bytes ? bytes : 16)); return MT_OK; }
int mt_host_free(void* ptr) { MT_CHECK_CUDA(cudaFreeHost(ptr)); return MT_OK; }
int mt_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
  MT_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return MT_OK;
}
int mt_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
  MT_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return MT_OK;
}
int mt_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
  MT_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
  return MT_OK;
}
int mt_memset(void* dst, int byte, size_t bytes, void* stream) {
  MT_CHECK_CUDA(cudaMemsetAsync(dst, byte, bytes, as_stream(stream)));
  return MT_OK;
}
int mt_stream_create(void** stream) {
  cudaStream_t s;
  MT_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return MT_OK;
}
int mt_stream_destroy(void* stream) { MT_CHECK_CUDA(cudaStreamDestroy(as_stream(stream))); return MT_OK; }
int mt_stream_sync(void* stream) { MT_CHECK_CUDA(cudaStreamSynchronize(as_stream(stream))); return MT_OK; }
int mt_device_sync(void) { MT_CHECK_CUDA(cudaDeviceSynchronize()); return MT_OK; }
int mt_event_create(void** event) {
  cudaEvent_t e;
  MT_CHECK_CUDA(cudaEventCreate(&e));
  *event = e;
  return MT_OK;
}
int mt_event_destroy(void* event) { MT_CHECK_CUDA(cudaEventDestroy((cudaEvent_t)event)); return MT_OK; }
int mt_event_record(void* event, void* stream) { MT_CHECK_CUDA(cudaEventRecord((cudaEvent_t)event, as_stream(stream))); return MT_OK; }
int mt_event_sync(void* event) { MT_CHECK_CUDA(cudaEventSynchronize((cudaEvent_t)event)); return MT_OK; }
int mt_event_elapsed_ms(void* start, void* stop, float* ms) {
  MT_CHECK_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return MT_OK;
}
int mt_stream_wait_event(void* stream, void* event) {
  MT_CHECK_CUDA(cudaStreamWaitEvent(as_stream(stream), (cudaEvent_t)event, 0));
  return MT_OK;
}
int mt_mem_info(size_t* free_bytes, size_t* total_bytes) {
  MT_CHECK_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
  return MT_OK;
}

int mt_device_flag_read(int* flag, void* stream) {
  int* p = device_flag_ptr();
  if (!p) { set_error("no device status word"); return MT_ERR_CUDA; }
  MT_CHECK_CUDA(cudaMemcpyAsync(flag, p, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream)));
  MT_CHECK_CUDA(cudaMemsetAsync(p, 0, sizeof(int), as_stream(stream)));
  MT_CHECK_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return MT_OK;
}

int mt_prof_begin(int kind) {
  for (auto& r : g_prof) g_prof_free.push_back(r);
  g_prof.clear();
  g_prof_kind = kind;
  return MT_OK;
}
int mt_prof_end(double* total_ms, int64_t* launches, double* total_flops) {
  double ms = 0, fl = 0;
  g_prof_kind = 0;
  for (auto& r : g_prof) {
    MT_CHECK_CUDA(cudaEventSynchronize(r.b));
    float t = 0;
    MT_CHECK_CUDA(cudaEventElapsedTime(&t, r.a, r.b));
    ms += t;
    fl += r.flops;
  }
  *total_ms = ms;
  *launches = (int64_t)g_prof.size();
  *total_flops = fl;
  for (auto& r : g_prof) g_prof_free.push_back(r);
  g_prof.clear();
  return MT_OK;
}

}  // extern "C"
