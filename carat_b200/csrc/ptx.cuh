// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarriers, TMA tile loads
// (cp.async.bulk.tensor, never with cluster multicast), tcgen05 MMA / TMEM management.
//
// Every wait in this file is bounded: a wait that runs out returns false, and the caller records
// an error word the host reads after the launch instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace carat_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbarrier_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbarrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbarrier_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.b32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  return done != 0;
}

// Roughly two seconds at 2 GHz. Generous for any real wait, short enough that a broken pipeline
// returns control to the host with an error word instead of hanging the device.
constexpr long long wait_cycle_limit = 4000000000LL;

__device__ __forceinline__ bool mbarrier_wait_bounded(uint32_t bar, uint32_t parity,
                                                      long long cycle_limit = wait_cycle_limit) {
  if (mbarrier_try_wait(bar, parity))
    return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 256; ++spin) {
      if (mbarrier_try_wait(bar, parity))
        return true;
    }
    if (clock64() - start > cycle_limit)
      return false;
  }
}

// The same wait for single-thread issue loops, where every instruction of the loop body is on the
// critical path: the common case (the phase has already completed) costs one try_wait.
__device__ __forceinline__ bool mbarrier_wait_fast(uint32_t bar, uint32_t parity) {
  if (mbarrier_try_wait(bar, parity))
    return true;
  return mbarrier_wait_bounded(bar, parity);
}

// Bounded wait for kernels with several roles: gives up at once when another role of the CTA has
// already given up (`abort_flag`, in shared memory), otherwise waits, and on running out records
// `code` in the per-device error word and raises the flag. The common case (the phase has
// completed) costs a single try_wait.
__device__ __forceinline__ bool mbarrier_wait_checked(uint32_t bar, uint32_t parity,
                                                      volatile int *abort_flag, int *device_error,
                                                      int code,
                                                      long long cycle_limit = wait_cycle_limit) {
  if (mbarrier_try_wait(bar, parity))
    return true;
  if (*abort_flag != 0)
    return false;
  if (mbarrier_wait_bounded(bar, parity, cycle_limit))
    return true;
  *abort_flag = 1;
  atomicExch(device_error, code);
  return false;
}

// One lane of a converged warp (the same one every time) gets true.
__device__ __forceinline__ bool elect_one() {
  uint32_t elected;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "elect.sync _|p, 0xFFFFFFFF;\n\t"
               "selp.b32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(elected));
  return elected != 0;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tile load into this CTA's shared memory; completion is signalled on `bar` as transaction
// bytes. x is the innermost (contiguous) coordinate and must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
               ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
               : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            int z, uint32_t bar, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
               ".L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
               : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
// Whole-warp call. Writes the TMEM base address (lane 0, first column) to `smem_result`.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_thread_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_thread_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrives on `bar` once every tcgen05.mma this thread issued before it has completed.
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T for 8-bit float operands (e4m3 here), K = 32 per instruction.
__device__ __forceinline__ void tcgen05_mma_f8f6f4(uint32_t tmem_d, uint64_t desc_a,
                                                   uint64_t desc_b, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(tmem_d),
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Same for 16-bit operands (bf16 here), K = 16 per instruction.
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(tmem_d),
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Variants for issue loops. The descriptors travel as 32-bit halves so that stepping along K or to
// the next pipeline stage is one 32-bit add on the low word (the start-address field; it cannot
// carry into the neighbouring field while the tile stays inside shared memory), and the
// accumulate flag is usually a constant the compiler folds.
__device__ __forceinline__ void tcgen05_mma_f16_split(uint32_t tmem_d, uint32_t a_low,
                                                      uint32_t a_high, uint32_t b_low,
                                                      uint32_t b_high, uint32_t idesc,
                                                      uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               ".reg .b64 da, db;\n\t"
               "setp.ne.b32 p, %6, 0;\n\t"
               "mov.b64 da, {%1, %2};\n\t"
               "mov.b64 db, {%3, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
               "}" ::"r"(tmem_d),
               "r"(a_low), "r"(a_high), "r"(b_low), "r"(b_high), "r"(idesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void tcgen05_mma_f8f6f4_split(uint32_t tmem_d, uint32_t a_low,
                                                         uint32_t a_high, uint32_t b_low,
                                                         uint32_t b_high, uint32_t idesc,
                                                         uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               ".reg .b64 da, db;\n\t"
               "setp.ne.b32 p, %6, 0;\n\t"
               "mov.b64 da, {%1, %2};\n\t"
               "mov.b64 db, {%3, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t"
               "}" ::"r"(tmem_d),
               "r"(a_low), "r"(a_high), "r"(b_low), "r"(b_high), "r"(idesc), "r"(accumulate)
               : "memory");
}

// The same with the A operand in tensor memory: lane = A row (M = 128), each 32-bit column holds
// two consecutive K elements, so one instruction (K = 16) consumes eight columns from `tmem_a`.
__device__ __forceinline__ void tcgen05_mma_f16_tmem_a(uint32_t tmem_d, uint32_t tmem_a,
                                                       uint32_t b_low, uint32_t b_high,
                                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               ".reg .b64 db;\n\t"
               "setp.ne.b32 p, %5, 0;\n\t"
               "mov.b64 db, {%2, %3};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
               "}" ::"r"(tmem_d),
               "r"(tmem_a), "r"(b_low), "r"(b_high), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Each thread of the warp writes 32 registers to 32 consecutive columns of its own TMEM lane.
__device__ __forceinline__ void tmem_store_32x32b_x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
      "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31])
      : "memory");
}

__device__ __forceinline__ void tmem_store_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Each thread of the warp reads 32 consecutive fp32 columns of its own TMEM lane
// (lane = 32 * (warp % 4) + laneid).
__device__ __forceinline__ void tmem_load_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
                 "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                 "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile written by TMA with the 128-byte
// swizzle: rows are 128 bytes, eight rows form one 1024-byte swizzle atom, so the stride between
// 8-row groups (SBO) is 1024 bytes; the leading-dimension field is 1 (ignored for swizzled
// K-major). Bits 46-47 carry descriptor version 1 (sm_100); bits 61-63 the layout (2 = 128B).
// The tile base must be 1024-byte aligned; advancing along K inside the atom adds the byte
// offset (32 per UMMA K step of 8-bit data) to the start address.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_address) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3FFFFU) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// MN-major operand written by TMA as [rows = K index][64 elements = MN index] with the 128-byte
// swizzle: eight K rows form one 1024-byte atom (SBO), the next 64 MN elements live in the next
// TMA box `mn_atom_bytes` further (LBO).
__device__ __forceinline__ uint64_t umma_desc_mn_major_sw128(uint32_t smem_address,
                                                             uint32_t mn_atom_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3FFFFU) >> 4);
  desc |= static_cast<uint64_t>(mn_atom_bytes >> 4) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// Instruction descriptor: fp32 accumulate, both operands K-major, no negate, dense.
// format codes: kind::f8f6f4 0 = e4m3; kind::f16 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t a_format, uint32_t b_format, uint32_t m,
                                                  uint32_t n) {
  return (1U << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

} // namespace ptx
} // namespace carat_b200
