// Thin wrappers over the sm_100a PTX this library issues by hand: mbarrier, bulk
// asynchronous copies (TMA unit, untiled form), tensor-memory management, tcgen05 MMA,
// tensor-memory loads/stores, and the fences between the generic and async proxies.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace akl {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// An mbarrier object must be invalidated before its memory is initialised again.
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// ---- bulk copy global -> shared, completion on an mbarrier ------------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- proxies / fences -------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- per-warpgroup register re-budgeting ------------------------------------------
// All four warps of a warpgroup execute the same instruction.  `inc` waits until the CTA's pool
// holds enough registers that other warpgroups released with `dec`; the budgets must add up.
template <int kRegs>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---- tensor memory ----------------------------------------------------------
// One warp, all lanes.  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Shared-memory operand descriptor, K-major, 128-byte swizzle: rows of 128 bytes, eight
// rows per 1024-byte swizzle atom (stride-byte-offset 1024), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}

// Instruction descriptor for kind::f8f6f4 with E4M3 A and B (both K-major), fp32 D.
__host__ __device__ constexpr uint32_t idesc_e4m3(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Instruction descriptor for kind::i8 with signed 8-bit A and B (both K-major), s32 D.
__host__ __device__ constexpr uint32_t idesc_s8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T ; one thread issues.
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// Same with INT8 operands and an exact s32 accumulator.
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// Arrive on an mbarrier when every tcgen05 operation this thread issued so far is done.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

#define AKL_R8(v, o) "=r"(v[o + 0]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), "=r"(v[o + 5]), "=r"(v[o + 6]), "=r"(v[o + 7])
#define AKL_I8(v, o) "r"(v[o + 0]), "r"(v[o + 1]), "r"(v[o + 2]), "r"(v[o + 3]), "r"(v[o + 4]), "r"(v[o + 5]), "r"(v[o + 6]), "r"(v[o + 7])

// Lane i of the calling warp reads 32 consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : AKL_R8(v, 0), AKL_R8(v, 8), AKL_R8(v, 16), AKL_R8(v, 24)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::AKL_I8(v, 0), AKL_I8(v, 8), AKL_I8(v, 16), AKL_I8(v, 24), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32 pairs: one issue slot for two IEEE round-to-nearest operations, bit-identical to
// the scalar forms.
__device__ __forceinline__ void mul2(float& a, float& b, float s) {          // a *= s; b *= s
  asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %2};\n\t"
      "mul.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a), "+f"(b) : "f"(s));
}
__device__ __forceinline__ void fma2(float& a, float& b, float m, float c) {  // a = a*m + c; b = b*m + c
  asm("{\n\t.reg .b64 x, y, z;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %2};\n\tmov.b64 z, {%3, %3};\n\t"
      "fma.rn.f32x2 x, x, y, z;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a), "+f"(b) : "f"(m), "f"(c));
}
__device__ __forceinline__ void add2(float& a, float& b, float x, float y) {  // a += x; b += y
  asm("{\n\t.reg .b64 p, q;\n\tmov.b64 p, {%0, %1};\n\tmov.b64 q, {%2, %3};\n\t"
      "add.rn.f32x2 p, p, q;\n\tmov.b64 {%0, %1}, p;\n\t}"
      : "+f"(a), "+f"(b) : "f"(x), "f"(y));
}

// max(a, b, c) in one instruction (three-input form of sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for two values on the FMA pipe (no MUFU): x = n + f with n = round(x), f in [-0.5, 0.5];
// 2^f by a degree-5 polynomial (relative error 2.3e-7, the class of ex2.approx), scaled by 2^n
// through an integer add into the exponent field.  Needs -125 <= x < 128; callers clamp.
__device__ __forceinline__ void exp2_poly2(float& a, float& b) {
  asm("{\n\t.reg .b64 x, t, n, f, p, c;\n\t.reg .b32 t0, t1, p0, p1;\n\t"
      "mov.b64 x, {%0, %1};\n\t"
      "mov.b64 c, {%2, %2};\n\t"
      "add.rn.f32x2 t, x, c;\n\t"          // low mantissa bits of t hold n
      "sub.rn.f32x2 n, t, c;\n\t"
      "sub.rn.f32x2 f, x, n;\n\t"
      "mov.b64 p, {%3, %3};\n\t"
      "mov.b64 c, {%4, %4};\n\tfma.rn.f32x2 p, p, f, c;\n\t"
      "mov.b64 c, {%5, %5};\n\tfma.rn.f32x2 p, p, f, c;\n\t"
      "mov.b64 c, {%6, %6};\n\tfma.rn.f32x2 p, p, f, c;\n\t"
      "mov.b64 c, {%7, %7};\n\tfma.rn.f32x2 p, p, f, c;\n\t"
      "mov.b64 c, {%8, %8};\n\tfma.rn.f32x2 p, p, f, c;\n\t"
      "mov.b64 {p0, p1}, p;\n\tmov.b64 {t0, t1}, t;\n\t"
      "shl.b32 t0, t0, 23;\n\tshl.b32 t1, t1, 23;\n\t"
      "add.s32 p0, p0, t0;\n\tadd.s32 p1, p1, t1;\n\t"
      "mov.b32 %0, p0;\n\tmov.b32 %1, p1;\n\t}"
      : "+f"(a), "+f"(b)
      : "f"(12582912.0f), "f"(0.0013276288518682122f), "f"(0.009675540030002594f), "f"(0.05550713837146759f),
        "f"(0.24022120237350464f), "f"(0.6931469440460205f), "f"(1.0000001192092896f));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace ptx
}  // namespace akl
