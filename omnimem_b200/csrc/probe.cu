// Measurement aid, not part of the selection path: the rate at which one thread block per SM can pull
// bulk copies into shared memory in the streaming dK/dV kernel's shape (4 stages of three 16 KiB
// copies, one issuing thread, nothing computed).  bench.py times it over a buffer that fits L2 and
// over one that does not; the two rates are the delivery rooflines quoted for that kernel.
#include "common.cuh"
#include "tc_common.cuh"

namespace nsa {
int device_status_address(int32_t** out);
namespace {
using namespace tc;

constexpr int kStages = 4, kPerStage = 3;
constexpr uint32_t kChunk = 16384;

__global__ void __launch_bounds__(64, 1)
bulk_stream_kernel(const char* __restrict__ buf, size_t items, int passes, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full[kStages], empty[kStages];
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort = &s_abort;
  // item i = chunk i of each of the buffer's three thirds: every byte of the buffer once per pass
  if (threadIdx.x == 0) {
    uint32_t it = 0;
    for (int p = 0; p < passes && !*abort; ++p)
      for (size_t i = blockIdx.x; i < items; i += gridDim.x, ++it) {
        const int st = it % kStages;
        if (it >= kStages && !mbar_wait(&empty[st], ((it / kStages) & 1) ^ 1, abort)) break;
        mbar_expect_tx(&full[st], kChunk * kPerStage);
        for (int c = 0; c < kPerStage; ++c)
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(tiles + (st * kPerStage + c) * kChunk)), "l"(buf + (c * items + i) * kChunk), "r"(kChunk),
                         "r"(smem_u32(&full[st])) : "memory");
      }
  } else if (threadIdx.x == 32) {
    uint32_t it = 0;
    bool ok = true;
    for (int p = 0; p < passes && ok; ++p)
      for (size_t i = blockIdx.x; i < items; i += gridDim.x, ++it) {
        const int st = it % kStages;
        if (!(ok = mbar_wait(&full[st], (it / kStages) & 1, abort))) break;    // every copy issued is waited for here
        mbar_arrive(&empty[st]);
      }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_abort) atomicExch(status, NSA_ERR_CUDA);
}

}  // namespace
}  // namespace nsa

extern "C" int nsa_probe_bulk_stream(const void* buf, size_t bytes, int32_t passes, void* stream) {
  using namespace nsa;
  NSA_REQUIRE(buf != nullptr && aligned16(buf) && passes >= 1, NSA_ERR_INVALID, "probe_bulk_stream: bad arguments");
  const size_t items = bytes / (static_cast<size_t>(kChunk) * kPerStage);
  NSA_REQUIRE(items >= 1, NSA_ERR_INVALID, "probe_bulk_stream: buffer smaller than one item (48 KiB)");
  int dev = 0, sms = 0;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int32_t* status;
  int rc;
  if ((rc = device_status_address(&status))) return rc;
  const size_t smem = static_cast<size_t>(kStages) * kPerStage * kChunk + 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(bulk_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  bulk_stream_kernel<<<sms, 64, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const char*>(buf), items, passes, status);
  NSA_LAUNCH_OK("bulk_stream_kernel");
  return NSA_OK;
}
