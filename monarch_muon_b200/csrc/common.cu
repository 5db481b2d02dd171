// Error reporting, device queries and the device status word.
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace mmb {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

static thread_local const float* t_grad_scale = nullptr;
const float* device_grad_scale() { return t_grad_scale; }
void set_device_grad_scale(const float* p) { t_grad_scale = p; }

// Launch options are per host thread, like the error text and the gradient scale: two optimizers stepping on
// two threads do not see each other's settings.
static thread_local int t_sm_limit = 0;
void set_sm_limit(int n) { t_sm_limit = n < 0 ? 0 : n; }

static thread_local int t_gemm_dynamic = 0;
void set_gemm_schedule_dynamic(bool on) { t_gemm_dynamic = on ? 1 : 0; }
bool gemm_schedule_dynamic() { return t_gemm_dynamic != 0; }

static thread_local int t_gemm_dependent_launch = 1;
void set_gemm_dependent_launch(bool on) { t_gemm_dependent_launch = on ? 1 : 0; }
bool gemm_dependent_launch() { return t_gemm_dependent_launch != 0; }

static thread_local int t_stream_ctas_per_sm = 0;
// at most 32: scratch arrays of the reductions are sized for 32 CTAs per SM
void set_stream_ctas_per_sm(int n) { t_stream_ctas_per_sm = n < 0 ? 0 : (n > 32 ? 32 : n); }
bool stream_kernels_share_sms() { return t_stream_ctas_per_sm > 0; }
long long stream_grid_cap(int sms) {
  const int n = t_stream_ctas_per_sm;
  return static_cast<long long>(sms) * (n > 0 ? n : 32);
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_sms = 0;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev != cached_dev) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached_dev = dev;
    cached_sms = sms;
  }
  const int limit = t_sm_limit;
  if (limit > 0 && limit < cached_sms) return limit;
  return cached_sms;
}

}  // namespace mmb

extern "C" {

int mmb_version(void) { return 100; }

int mmb_set_device_grad_scale(const float* scale_dev) {
  mmb::set_device_grad_scale(scale_dev);
  return MMB_OK;
}

int mmb_set_sm_limit(int n) {
  mmb::set_sm_limit(n);
  return MMB_OK;
}

int mmb_set_stream_ctas_per_sm(int n) {
  using namespace mmb;
  MMB_REQUIRE(n >= 0 && n <= 32, "mmb_set_stream_ctas_per_sm: n = %d is outside 0..32", n);
  set_stream_ctas_per_sm(n);
  return MMB_OK;
}

int mmb_set_gemm_schedule(int dynamic) {
  mmb::set_gemm_schedule_dynamic(dynamic != 0);
  return MMB_OK;
}

int mmb_set_gemm_dependent_launch(int on) {
  mmb::set_gemm_dependent_launch(on != 0);
  return MMB_OK;
}

int64_t mmb_launch_count(void) { return mmb::launches(); }

const char* mmb_last_error(void) { return mmb::error_buffer(); }

int mmb_device_status_create(int32_t** status_dev_out) {
  using namespace mmb;
  MMB_REQUIRE(status_dev_out != nullptr, "mmb_device_status_create: null output");
  int32_t* p = nullptr;
  MMB_CUDA_CHECK(cudaMalloc(&p, 4 * sizeof(int32_t)));
  MMB_CUDA_CHECK(cudaMemset(p, 0, 4 * sizeof(int32_t)));
  *status_dev_out = p;
  return MMB_OK;
}

int mmb_device_status_destroy(int32_t* status_dev) {
  using namespace mmb;
  if (status_dev != nullptr) MMB_CUDA_CHECK(cudaFree(status_dev));
  return MMB_OK;
}

int mmb_device_status_read(int32_t* status_dev, int32_t* host_out, int reset, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(status_dev != nullptr && host_out != nullptr, "mmb_device_status_read: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MMB_CUDA_CHECK(cudaMemcpyAsync(host_out, status_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  if (reset) MMB_CUDA_CHECK(cudaMemsetAsync(status_dev, 0, 4 * sizeof(int32_t), st));
  MMB_CUDA_CHECK(cudaStreamSynchronize(st));
  return MMB_OK;
}

}  // extern "C"
