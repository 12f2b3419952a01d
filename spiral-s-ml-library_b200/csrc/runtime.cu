// Runtime shim of libspiral_b200: error text, device selection, memory,
// streams, events and the device status word.  It stands where the reference
// relies on CuPy for allocation, copies and synchronisation
// (corecuda/cupy.spi:20-58, corecuda/base.spi:45).
#include "common.cuh"

#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

static thread_local char t_error[512] = "";

static std::atomic<unsigned long long> g_sb_launch_count{0};
void sb_count_launch() { g_sb_launch_count.fetch_add(1, std::memory_order_relaxed); }

int sb_sm_count() {
  static std::atomic<int> sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SB_NUM_SMS_FALLBACK;
  int v = sms[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = SB_NUM_SMS_FALLBACK;
    sms[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

namespace {
constexpr int PROF_MAX = 4096;
// The GEMM profile is one process-wide recording: begin/end and the per-launch hooks take this lock,
// so launches from several host threads are recorded whole (in the order the lock is won).
std::mutex g_prof_lock;
bool g_prof_on = false;
int g_prof_n = 0;
cudaEvent_t g_prof_ev[2 * PROF_MAX];
bool g_prof_ev_made = false;
double g_prof_flops[PROF_MAX];
float g_prof_ms[PROF_MAX];
int g_prof_last_n = 0;
}  // namespace

bool sb_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB_NO_PDL");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}

// before/after bracket one launch: `before` takes the lock when a profile is being recorded and
// `after` releases it, so two threads' event pairs cannot interleave.
static thread_local bool t_prof_held = false;

void sb_prof_before(cudaStream_t s) {
  if (!g_prof_on) return;
  g_prof_lock.lock();
  if (!g_prof_on || g_prof_n >= PROF_MAX) {
    g_prof_lock.unlock();
    return;
  }
  t_prof_held = true;
  cudaEventRecord(g_prof_ev[2 * g_prof_n], s);
}

void sb_prof_after(cudaStream_t s, double flops) {
  if (!t_prof_held) return;
  cudaEventRecord(g_prof_ev[2 * g_prof_n + 1], s);
  g_prof_flops[g_prof_n] = flops;
  ++g_prof_n;
  t_prof_held = false;
  g_prof_lock.unlock();
}

void sb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int sb_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}

int sb_check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return SB_OK;
  int code = (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? SB_ERR_NO_DEVICE
                                                                           : SB_ERR_CUDA;
  return sb_fail(code, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

extern "C" {

const char* sb_last_error_string(void) { return t_error; }

int sb_version(void) { return 100; }

int sb_device_count(int* count) {
  if (!count) return sb_fail(SB_ERR_BAD_ARG, "sb_device_count: null output");
  *count = 0;
  cudaError_t e = cudaGetDeviceCount(count);
  if (e != cudaSuccess) {
    *count = 0;
    return sb_check_cuda(e, "cudaGetDeviceCount");
  }
  return SB_OK;
}

int sb_set_device(int device) {
  SB_CUDA(cudaSetDevice(device));
  return SB_OK;
}

int sb_device_sm_count(int* sms) {
  if (!sms) return sb_fail(SB_ERR_BAD_ARG, "sb_device_sm_count: null output");
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  SB_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
  return SB_OK;
}

int sb_malloc(void** ptr, size_t bytes) {
  if (!ptr) return sb_fail(SB_ERR_BAD_ARG, "sb_malloc: null output");
  *ptr = nullptr;
  if (bytes == 0) bytes = 16;
  SB_CUDA(cudaMalloc(ptr, bytes));
  return SB_OK;
}

int sb_free(void* ptr) {
  if (!ptr) return SB_OK;
  SB_CUDA(cudaFree(ptr));
  return SB_OK;
}

int sb_malloc_host(void** ptr, size_t bytes) {
  if (!ptr) return sb_fail(SB_ERR_BAD_ARG, "sb_malloc_host: null output");
  *ptr = nullptr;
  if (bytes == 0) bytes = 16;
  SB_CUDA(cudaMallocHost(ptr, bytes));
  return SB_OK;
}

int sb_free_host(void* ptr) {
  if (!ptr) return SB_OK;
  SB_CUDA(cudaFreeHost(ptr));
  return SB_OK;
}

int sb_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return SB_OK;
  if (!dst || !src) return sb_fail(SB_ERR_BAD_ARG, "sb_memcpy_h2d: null pointer");
  SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return SB_OK;
}

int sb_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return SB_OK;
  if (!dst || !src) return sb_fail(SB_ERR_BAD_ARG, "sb_memcpy_d2h: null pointer");
  SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return SB_OK;
}

int sb_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return SB_OK;
  if (!dst || !src) return sb_fail(SB_ERR_BAD_ARG, "sb_memcpy_d2d: null pointer");
  SB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return SB_OK;
}

int sb_memset(void* dst, int value, size_t bytes, void* stream) {
  if (bytes == 0) return SB_OK;
  if (!dst) return sb_fail(SB_ERR_BAD_ARG, "sb_memset: null pointer");
  SB_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
  return SB_OK;
}

int sb_stream_create(void** stream) {
  if (!stream) return sb_fail(SB_ERR_BAD_ARG, "sb_stream_create: null output");
  cudaStream_t s;
  SB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = (void*)s;
  return SB_OK;
}

int sb_stream_destroy(void* stream) {
  if (!stream) return SB_OK;
  SB_CUDA(cudaStreamDestroy((cudaStream_t)stream));
  return SB_OK;
}

int sb_stream_sync(void* stream) {
  SB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return SB_OK;
}

int sb_device_sync(void) {
  SB_CUDA(cudaDeviceSynchronize());
  return SB_OK;
}

int sb_event_create(void** event) {
  if (!event) return sb_fail(SB_ERR_BAD_ARG, "sb_event_create: null output");
  cudaEvent_t e;
  SB_CUDA(cudaEventCreate(&e));
  *event = (void*)e;
  return SB_OK;
}

int sb_event_destroy(void* event) {
  if (!event) return SB_OK;
  SB_CUDA(cudaEventDestroy((cudaEvent_t)event));
  return SB_OK;
}

int sb_event_record(void* event, void* stream) {
  if (!event) return sb_fail(SB_ERR_BAD_ARG, "sb_event_record: null event");
  SB_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
  return SB_OK;
}

int sb_stream_wait_event(void* stream, void* event) {
  if (!event) return sb_fail(SB_ERR_BAD_ARG, "sb_stream_wait_event: null event");
  SB_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
  return SB_OK;
}

int sb_event_elapsed_ms(void* start, void* stop, float* ms) {
  if (!start || !stop || !ms) return sb_fail(SB_ERR_BAD_ARG, "sb_event_elapsed_ms: null argument");
  SB_CUDA(cudaEventSynchronize((cudaEvent_t)stop));
  SB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return SB_OK;
}

unsigned long long sb_launch_count(void) { return g_sb_launch_count.load(std::memory_order_relaxed); }

int sb_mem_info(size_t* free_bytes, size_t* total_bytes) {
  if (!free_bytes || !total_bytes) return sb_fail(SB_ERR_BAD_ARG, "sb_mem_info: null output");
  SB_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
  return SB_OK;
}

int sb_gemm_profile_begin(void) {
  std::lock_guard<std::mutex> hold(g_prof_lock);
  if (!g_prof_ev_made) {
    for (int i = 0; i < 2 * PROF_MAX; ++i) SB_CUDA(cudaEventCreate(&g_prof_ev[i]));
    g_prof_ev_made = true;
  }
  g_prof_n = 0;
  g_prof_on = true;
  return SB_OK;
}

int sb_gemm_profile_end(int* launches, double* total_ms, double* total_flops) {
  std::lock_guard<std::mutex> hold(g_prof_lock);
  g_prof_on = false;
  double ms = 0.0, fl = 0.0;
  for (int i = 0; i < g_prof_n; ++i) {
    SB_CUDA(cudaEventSynchronize(g_prof_ev[2 * i + 1]));
    float t = 0.f;
    SB_CUDA(cudaEventElapsedTime(&t, g_prof_ev[2 * i], g_prof_ev[2 * i + 1]));
    g_prof_ms[i] = t;
    ms += t;
    fl += g_prof_flops[i];
  }
  if (launches) *launches = g_prof_n;
  if (total_ms) *total_ms = ms;
  if (total_flops) *total_flops = fl;
  g_prof_last_n = g_prof_n;
  g_prof_n = 0;
  return SB_OK;
}

int sb_gemm_profile_entry(int index, double* ms, double* flops) {
  std::lock_guard<std::mutex> hold(g_prof_lock);
  if (index < 0 || index >= g_prof_last_n || !ms || !flops)
    return sb_fail(SB_ERR_BAD_ARG, "sb_gemm_profile_entry: index %d outside the last profile of %d launches", index, g_prof_last_n);
  *ms = g_prof_ms[index];
  *flops = g_prof_flops[index];
  return SB_OK;
}

int sb_device_status(int* status2, int clear) {
  if (!status2) return sb_fail(SB_ERR_BAD_ARG, "sb_device_status: null output");
  int host[4] = {0, 0, 0, 0};
  SB_CUDA(cudaDeviceSynchronize());
  SB_CUDA(cudaMemcpyFromSymbol(host, g_sb_status, sizeof(host)));
  status2[0] = host[0];
  status2[1] = host[1];
  if (clear && (host[0] != 0 || host[1] != 0)) {
    int zero[4] = {0, 0, 0, 0};
    SB_CUDA(cudaMemcpyToSymbol(g_sb_status, zero, sizeof(zero)));
  }
  return SB_OK;
}

int sb_check_device(void* stream) {
  SB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  int host[4] = {0, 0, 0, 0};
  SB_CUDA(cudaMemcpyFromSymbol(host, g_sb_status, sizeof(host)));
  if (host[0] != 0 || host[1] != 0)
    return sb_fail(SB_ERR_DEVICE_TIMEOUT,
                   "a bounded device-side wait expired (first wait site %d, %d waits in all): the kernels that were "
                   "running gave up and their outputs are incomplete; read the details with sb_device_status",
                   host[0], host[1]);
  return SB_OK;
}

}  // extern "C"
