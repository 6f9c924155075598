// Shared device helpers: operator geometry, PTX wrappers for mbarrier / TMA / tcgen05, bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/b200moe.h"

namespace b200moe {

constexpr int H = B200MOE_HIDDEN;        // 7168
constexpr int I = B200MOE_INTER;         // 2048
constexpr int E_GLOBAL = B200MOE_NUM_EXPERTS;
constexpr int TOP_K = B200MOE_TOP_K;
constexpr int N_GROUP = B200MOE_N_GROUP;
constexpr int TOPK_GROUP = B200MOE_TOPK_GROUP;
constexpr int QBLOCK = B200MOE_QBLOCK;
constexpr int BLOCK_M = B200MOE_BLOCK_M;
constexpr int H_BLOCKS = H / QBLOCK;     // 56
constexpr int I_BLOCKS = I / QBLOCK;     // 16

// Status codes written to workspace.status[0]; status[1..3] carry (blockIdx, role, detail).
constexpr int ST_OK = 0;
constexpr int ST_WAIT_TIMEOUT = 1;

// ---------------------------------------------------------------------------------------------------------
// Shared-memory / barrier PTX
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrival that orders nothing: for hand-backs where no memory written by this thread is read by the waiter (a TMEM stage
// whose columns are already in registers: tcgen05.wait::ld + tcgen05.fence::before_thread_sync).  The default arrival
// has release semantics, and a release waits for the thread's memory operations in flight: with the next chunk's scale
// loads under way it reached the barrier ~600 cycles after the warp had finished reading TMEM (cycle stamps), which held
// the tensor pipe at ~50 % duty.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll of a barrier phase.  The instruction may park the thread in hardware until the phase completes or
// B200MOE_WAIT_HINT_NS nanoseconds have passed, whichever comes first; completion wakes it at once.  Parked threads issue
// nothing, which matters here: the single-thread roles (TMA producer, MMA issuer) share their SM sub-partitions with the
// promotion warps, and a role that re-issued a failing poll every few cycles took enough issue slots to make the
// promotion warps on its sub-partition ~500 cycles late per 128-K chunk (cycle stamps: the warp next to the producer
// saw a completed barrier 850 cycles after the MMA issue, a warp on a quiet sub-partition after 350).
#ifndef B200MOE_WAIT_HINT_NS
#define B200MOE_WAIT_HINT_NS 20000
#endif
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
#if B200MOE_WAIT_HINT_NS > 0
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(static_cast<uint32_t>(B200MOE_WAIT_HINT_NS))
      : "memory");
#else
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
#endif
  return ok;
}
// Wait on an mbarrier phase with a time limit.  Returns false (and records why) instead of hanging: `abort_flag` is a
// CTA-shared word every waiting role looks at between polls, so one role giving up releases the others within one poll
// period.  The limit is counted on the SM's cycle counter, read only when a poll came back empty, so a healthy wait
// (microseconds) costs one instruction.
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // about 2 s at B200 clocks
// polls a giving-up role spends on each of its copies still in flight (each poll may take up to the hint)
constexpr int DRAIN_POLLS = B200MOE_WAIT_HINT_NS > 0 ? (1 << 14) : (1 << 20);
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int role, int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
#if B200MOE_WAIT_HINT_NS > 0
  constexpr uint32_t CHECK_MASK = 0x0;     // a failed poll already took up to the hint: check every time
#else
  constexpr uint32_t CHECK_MASK = 0x3ff;   // polls return at once: look at the clock every 1024 tries
#endif
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & CHECK_MASK) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      if (now - t0 > WAIT_LIMIT_CYCLES) {
        *abort_flag = 1;
        if (atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT) == ST_OK) {
          status[1] = static_cast<int>(blockIdx.x);
          status[2] = role;
          status[3] = detail;
        }
        return false;
      }
    }
  }
}

// A shared-memory counter as a one-way signal: the writers add with release ordering, one reader polls it with acquire
// loads until it reaches `target` (bounded like mbar_wait).  A poll is a plain shared-memory load: nothing parks, and
// the reader sees the last addition a few tens of cycles after it happens.
__device__ __forceinline__ void red_add_release_shared(uint32_t* counter, uint32_t v) {
  asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;"
               ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(counter))), "r"(v)
               : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_shared(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];"
               : "=r"(v)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p)))
               : "memory");
  return v;
}
__device__ __forceinline__ bool counter_wait(const uint32_t* counter, uint32_t target, volatile int* abort_flag,
                                             int* status, int role, int detail) {
  if (ld_acquire_shared(counter) >= target) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    if (ld_acquire_shared(counter) >= target) return true;
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > WAIT_LIMIT_CYCLES) {
        *abort_flag = 1;
        if (atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT) == ST_OK) {
          status[1] = static_cast<int>(blockIdx.x);
          status[2] = role;
          status[3] = detail;
        }
        return false;
      }
    }
  }
}

// Warp-level form: every lane polls and the warp agrees on the outcome (all lanes polling measured faster on B200
// than one elected lane with the rest parked at a warp barrier every time: 967 vs 1204 cycles per GEMM chunk; roles
// that only ever need one thread run their whole loop as lane 0 instead).
__device__ __forceinline__ bool mbar_wait_all(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                              int role, int detail) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, role, detail));
}

// ---------------------------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor, no multicast anywhere)
// ---------------------------------------------------------------------------------------------------------
// 16-byte asynchronous copy global -> shared through the load/store unit (not TMA), L2 only, with the neighbouring
// 128 bytes brought into L2 as well; groups, and the fence that makes such generic-proxy writes visible to the
// tensor core's (async-proxy) reads of shared memory.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Ask for the box to be brought into L2 only: no shared-memory destination, no completion to wait for.
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D tiled load: c0 = innermost (byte/element column, must be a multiple of 16 bytes), c1 = row.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// tcgen05 (5th-generation tensor core, TMEM accumulators)
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// mbarrier arrives (count 1) once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], e4m3 x e4m3 -> f32, issued by ONE thread.
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base+i), r[j] = column (col0+j).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 64 consecutive 32-bit columns in one instruction: thread i receives lane (base+i), r[j] = column (col0+j).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void setmaxnreg_inc_promo() { asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); }
__device__ __forceinline__ void setmaxnreg_dec_aux() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }
// Same pool split differently (one warpgroup at DEC, two at INC; 128 * DEC + 256 * INC <= 64512 registers).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }


// UMMA shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle
// (8-row x 128-byte atoms, 1024 bytes apart).  Bits: [0,14) address>>4, [16,30) leading byte offset>>4 (unused for
// swizzled K-major, set to 1), [32,46) stride byte offset>>4 (= 1024>>4), [46,48) version 1, [61,64) layout 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// UMMA instruction descriptor, kind::f8f6f4: D f32, A/B e4m3, both K-major, no negate, dense.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int m, int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------------------
// Small numeric helpers
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// Programmatic dependent launch: every kernel of the layer lets its successor be scheduled early
// (pdl_launch_dependents at entry) and blocks in pdl_wait until its predecessor has completed and flushed before it
// touches global memory.  Only launch latency and per-CTA set-up overlap; data dependences stay kernel-to-kernel.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Launch-side error helper used by the .cu files.
#define B200MOE_CUDA_TRY(expr)                                   \
  do {                                                           \
    cudaError_t _e = (expr);                                     \
    if (_e != cudaSuccess) return b200moe::record_cuda_error(_e); \
  } while (0)

int record_cuda_error(cudaError_t e);

}  // namespace b200moe
