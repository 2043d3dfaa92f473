// Library-wide pieces of the C ABI: error text, version, struct sizes, device properties.
#include "tc_common.cuh"

#include <string.h>
#include <atomic>

namespace qb {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

static std::atomic<int> g_early_overlap{0};
bool early_overlap() { return g_early_overlap.load(std::memory_order_relaxed) != 0; }

static std::atomic<int> g_sm_budget{0};

int device_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev < 64) cached[dev] = n;
  return n;
}

int sm_count() {
  const int n = device_sm_count(), cap = g_sm_budget.load(std::memory_order_relaxed);
  return cap > 0 && cap < n ? cap : n;
}

static std::atomic<int> g_path_override{0};
bool path_override(int bit) { return (g_path_override.load(std::memory_order_relaxed) & bit) != 0; }

static __device__ int g_device_status = 0;

int* device_status_ptr() {
  static int* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev < 64 && cached[dev] != nullptr) return cached[dev];
  int* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_device_status) != cudaSuccess) return nullptr;
  if (dev < 64) cached[dev] = p;
  return p;
}

}  // namespace qb

extern "C" int qb_read_device_status(void* stream) {
  int v = 0;
  cudaStream_t st = (cudaStream_t)stream;
  QB_CUDA_OK(cudaStreamSynchronize(st));
  int* p = qb::device_status_ptr();
  QB_REQUIRE(p != nullptr, QB_ERR_CUDA, "device status word unavailable");
  QB_CUDA_OK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    QB_CUDA_OK(cudaMemset(p, 0, sizeof(int)));
    if (v == 501) {
      qb::set_error("embedding_lookup met a token id outside the table (code %d)", v);
      return QB_ERR_INVALID_ARG;
    }
    qb::set_error("a bounded device-side wait expired (code %d)", v);
    return QB_ERR_TIMEOUT;
  }
  return QB_OK;
}

extern "C" int qb_set_path_override(int mask) {
  return qb::g_path_override.exchange(mask);
}

extern "C" int qb_set_early_overlap(int on) {
  return qb::g_early_overlap.exchange(on != 0 ? 1 : 0);
}

extern "C" int qb_set_sm_budget(int sms) {
  return qb::g_sm_budget.exchange(sms < 0 ? 0 : sms);
}

extern "C" const char* qb_last_error(void) { return qb::t_error; }

extern "C" int qb_abi_version(void) { return 1; }

extern "C" int64_t qb_sizeof(const char* name) {
  if (name == nullptr) return -1;
#define QB_SZ(T) if (strcmp(name, #T) == 0) return (int64_t)sizeof(T)
  QB_SZ(qb_conv1d_fwd_args);
  QB_SZ(qb_conv1d_update_args);
  QB_SZ(qb_quamba2_conv1d_fwd_args);
  QB_SZ(qb_quamba2_conv1d_update_args);
  QB_SZ(qb_hadamard_quant_args);
  QB_SZ(qb_sscan_fwd_args);
  QB_SZ(qb_sscan_update_args);
  QB_SZ(qb_ssd_args);
  QB_SZ(qb_w4a8_unpack_args);
  QB_SZ(qb_w4a8_gemm_args);
  QB_SZ(qb_w4a8_gemv_s4_args);
  QB_SZ(qb_w8a8_gemm_args);
  QB_SZ(qb_rmsnorm_args);
  QB_SZ(qb_embedding_args);
  QB_SZ(qb_decode_norm_linear_args);
  QB_SZ(qb_decode_gate_had_quant_args);
  QB_SZ(qb_peer_put_args);
#undef QB_SZ
  return -1;
}
