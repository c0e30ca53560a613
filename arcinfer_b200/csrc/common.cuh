// Shared device helpers for libarcsample (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/arcsample.h"

namespace arcs {

constexpr int kThreads = 256;          // threads per CTA of the streaming kernels
constexpr int kTileBytes = 16384;      // four 16-byte chunks per thread per tile
constexpr int kStages = 3;             // tiles in the bulk-copy ring of a CTA
constexpr uint32_t kWaitLimit = 1u << 22;  // bounded mbarrier wait (tries)

// ---------------------------------------------------------------- order-preserving keys
// float -> uint32 such that a < b  <=>  key(a) < key(b); -0 is folded into +0 (equal as
// floats) and NaN maps to 0, below every number, so it is never selected.
__device__ __forceinline__ uint32_t key_of(float v) {
  v = v + 0.0f;
  uint32_t b = __float_as_uint(v);
  if (v != v) return 0u;
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float value_of(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
// 64-bit composite: larger = better under (value descending, id ascending)
__device__ __forceinline__ uint64_t comp_of(uint32_t key, int32_t id) {
  return ((uint64_t)key << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)id);
}
__device__ __forceinline__ int32_t comp_id(uint64_t c) { return (int32_t)(0xFFFFFFFFu - (uint32_t)c); }
__device__ __forceinline__ uint32_t comp_key(uint64_t c) { return (uint32_t)(c >> 32); }

// ---------------------------------------------------------------- element access
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kPerChunk = 4;
  static __device__ __forceinline__ float load(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ float from_smem(const char* p) { return *reinterpret_cast<const float*>(p); }
  // value j of a 16-byte chunk
  static __device__ __forceinline__ float get(const uint4& q, int j) {
    return __uint_as_float(j == 0 ? q.x : j == 1 ? q.y : j == 2 ? q.z : q.w);
  }
  // maximum of the chunk ignoring NaN (fmaxf returns the other operand for a NaN)
  static __device__ __forceinline__ float chunk_max(const uint4& q) {
    return fmaxf(fmaxf(__uint_as_float(q.x), __uint_as_float(q.y)), fmaxf(__uint_as_float(q.z), __uint_as_float(q.w)));
  }
  // chunk-level threshold test: `thr` is made once from a float threshold by make_thr
  typedef float Thr;
  static __device__ __forceinline__ Thr make_thr(float t) { return t; }
  static __device__ __forceinline__ bool chunk_reaches(const uint4& q, Thr t) { return chunk_max(q) >= t; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kPerChunk = 8;
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) {
    return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p)) << 16);
  }
  static __device__ __forceinline__ float from_smem(const char* p) {
    return __uint_as_float((uint32_t)*reinterpret_cast<const unsigned short*>(p) << 16);
  }
  static __device__ __forceinline__ float get(const uint4& q, int j) {
    const uint32_t w = (j >> 1) == 0 ? q.x : (j >> 1) == 1 ? q.y : (j >> 1) == 2 ? q.z : q.w;
    return __uint_as_float((j & 1) ? (w & 0xFFFF0000u) : (w << 16));  // exact widening
  }
  static __device__ __forceinline__ float chunk_max(const uint4& q) {
    __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&q.x);
    __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
    __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&q.z);
    __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(&q.w);
    const __nv_bfloat162 m = __hmax2(__hmax2(a, b), __hmax2(c, d));  // NaN-ignoring packed max
    return fmaxf(__low2float(m), __high2float(m));
  }
  // chunk-level threshold test on packed pairs: the threshold is rounded DOWN to bf16, so the
  // test can only err on the side of listing a chunk
  typedef __nv_bfloat162 Thr;
  static __device__ __forceinline__ Thr make_thr(float t) { return __bfloat162bfloat162(__float2bfloat16_rd(t)); }
  static __device__ __forceinline__ bool chunk_reaches(const uint4& q, Thr t) {
    __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&q.x);
    __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
    __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&q.z);
    __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(&q.w);
    return __hge2_mask(__hmax2(__hmax2(a, b), __hmax2(c, d)), t) != 0u;
  }
};

// ---------------------------------------------------------------- warp helpers
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const uint64_t w = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = w > v ? w : v;
  }
  return v;
}

// ---------------------------------------------------------------- mbarrier + bulk copy (TMA, 1-D)
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// orders this thread's earlier generic-proxy accesses of shared memory before its later bulk copies
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// one arrival (of a barrier initialised with the number of arrivals a phase takes)
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// non-blocking test of a phase
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase did not complete within kWaitLimit tries (never seen in
// practice; the caller then raises ARCS_ERR_TIMEOUT instead of spinning forever).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 16) __nanosleep(it > 256 ? 256 : 32);  // (try_wait itself suspends the thread for a while)
  }
  return false;
}
// The same wait for a whole warp: every lane tries (one instruction for the warp; the hardware
// suspends the warp inside the try for a while, so that few tries are issued).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < kWaitLimit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion counted on `bar`. No multicast: the destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}


// ---------------------------------------------------------------- explicit shared-memory accesses
// Pointers that travel through structs or out-of-line functions lose their address space and
// compile to generic accesses; these helpers keep atomics and polled words on the shared path.
__device__ __forceinline__ uint32_t sm_atomic_add(void* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_addr(p)), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void sm_red_add(void* p, uint32_t v) {
  asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(smem_addr(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void sm_red_or(void* p, uint32_t v) {
  asm volatile("red.shared.or.b32 [%0], %1;" ::"r"(smem_addr(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void sm_red_min_s32(void* p, int32_t v) {
  asm volatile("red.shared.min.s32 [%0], %1;" ::"r"(smem_addr(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void sm_red_max_u64(void* p, unsigned long long v) {
  asm volatile("red.shared.max.u64 [%0], %1;" ::"r"(smem_addr(p)), "l"(v) : "memory");
}
__device__ __forceinline__ void sm_red_min_u64(void* p, unsigned long long v) {
  asm volatile("red.shared.min.u64 [%0], %1;" ::"r"(smem_addr(p)), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t sm_atomic_cas(void* p, uint32_t expect, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "r"(smem_addr(p)), "r"(expect), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t sm_ld_volatile(const void* p) {
  uint32_t v;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr(p)) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t sm_ld(const void* p) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr(p)));
  return v;
}
__device__ __forceinline__ unsigned long long sm_ld_volatile64(const void* p) {
  unsigned long long v;
  asm volatile("ld.volatile.shared.u64 %0, [%1];" : "=l"(v) : "r"(smem_addr(p)) : "memory");
  return v;
}
__device__ __forceinline__ void sm_st_volatile64(void* p, unsigned long long v) {
  asm volatile("st.volatile.shared.u64 [%0], %1;" ::"r"(smem_addr(p)), "l"(v) : "memory");
}

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while the kernel
// before it on the stream still runs; it must pass pdl_wait() before it touches anything that
// kernel writes (the wait returns when that kernel has completed and its writes are visible).
// pdl_trigger() in the earlier kernel lets the later one be scheduled as soon as there is room.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void raise_status(int32_t* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

}  // namespace arcs
