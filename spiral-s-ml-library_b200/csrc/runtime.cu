// Runtime shim of libspiral_b200: error text, device selection, memory,
// streams, events and the device status word.  It stands where the reference
// relies on CuPy for allocation, copies and synchronisation
// (corecuda/cupy.spi:20-58, corecuda/base.spi:45).
#include "common.cuh"

#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

static thread_local char t_error[512] = "";

unsigned long long g_sb_launch_count = 0;

namespace {
constexpr int PROF_MAX = 4096;
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

void sb_prof_before(cudaStream_t s) {
  if (!g_prof_on || g_prof_n >= PROF_MAX) return;
  cudaEventRecord(g_prof_ev[2 * g_prof_n], s);
}

void sb_prof_after(cudaStream_t s, double flops) {
  if (!g_prof_on || g_prof_n >= PROF_MAX) return;
  cudaEventRecord(g_prof_ev[2 * g_prof_n + 1], s);
  g_prof_flops[g_prof_n] = flops;
  ++g_prof_n;
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

unsigned long long sb_launch_count(void) { return g_sb_launch_count; }

int sb_gemm_profile_begin(void) {
  if (!g_prof_ev_made) {
    for (int i = 0; i < 2 * PROF_MAX; ++i) SB_CUDA(cudaEventCreate(&g_prof_ev[i]));
    g_prof_ev_made = true;
  }
  g_prof_n = 0;
  g_prof_on = true;
  return SB_OK;
}

int sb_gemm_profile_end(int* launches, double* total_ms, double* total_flops) {
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

}  // extern "C"
