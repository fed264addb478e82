// Inline-PTX wrappers for the sm_100a features the GEMM uses: mbarrier, TMA loads (every load lands in the
// shared memory of the CTA that issued it), tensor memory (tcgen05.alloc/ld/cp), the 5th-generation
// tensor-core MMA (tcgen05.mma kind::mxf8f6f4.block_scale) in its one-CTA and CTA-pair forms, and the
// cluster plumbing a CTA pair needs (rank, remote mbarrier arrive, cluster barrier). Device-only.
//
// The wrappers that issue asynchronous work (loads, copies, MMAs, commits, expect_tx) take `pred`: the whole warp
// executes the call converged and only the lane whose pred is non-zero (one elected lane) issues the instruction.
// Keeping the issuing warp converged lets the compiler hold descriptors and addresses in uniform registers;
// issuing from inside a divergent `if (lane == 0)` costs roughly twice the cycles per instruction, enough to make
// a 128 x 256 x 32 MMA stream issue-bound.
#pragma once

#include <cstdint>

#include <cuda.h>

namespace mxb200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t pred, uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}\n" ::"r"(smem_u32(bar)), "r"(bytes), "r"(pred)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
  return done != 0;
}

// Overloads taking the barrier as a shared-memory address (the issuing warps keep running addresses).
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar_addr, uint32_t parity) {
  uint32_t done;
  asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar_addr), "r"(parity)
        : "memory");
  return done != 0;
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t pred, uint32_t bar_addr, uint32_t bytes) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}\n" ::"r"(bar_addr), "r"(bytes), "r"(pred)
               : "memory");
}

// Generic-proxy writes to shared memory made visible to the async proxy (TMA stores, tcgen05 reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------- TMA

// 2-D tiled load global -> shared, completion on an mbarrier of this CTA. x is the innermost coordinate and
// must make x * element size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t pred, void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
        "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}\n"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(pred)
        : "memory");
}

// The same load with an L2 eviction-priority hint (a createpolicy value), for data that is read once.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t pred, void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                                 int32_t x, int32_t y, uint64_t policy) {
  asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
        "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %6;\n\t}\n"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(pred),
          "l"(policy)
        : "memory");
}

// Untiled bulk copy global -> shared: both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t pred, void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t"
        "@q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n\t}\n"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar)), "r"(pred)
        : "memory");
}

// 2-D tiled store shared -> global (bulk async-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y) {
  asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
        : "memory");
}

// The same with an L2 eviction-priority hint (a createpolicy value): output that this kernel never reads again should
// not push the operands out of L2.
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y,
                                                  uint64_t policy) {
  asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------------------------------------- tensor memory

// Whole-warp: allocate `cols` (a power of two >= 32) TMEM columns; the base address lands in *smem_out.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_out, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// All tcgen05.mma / tcgen05.cp issued so far by this thread arrive on the mbarrier when they complete.
__device__ __forceinline__ void tcgen05_commit(uint32_t pred, uint64_t* bar) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n"
               ::"r"(smem_u32(bar)), "r"(pred)
               : "memory");
}

// 32 rows x 16 bytes of shared memory (one 512-byte scale tile) -> TMEM lanes 0..31 x 4 columns, replicated
// into all four 32-lane quarters.
__device__ __forceinline__ void tcgen05_cp_32x128b_warpx4(uint32_t pred, uint32_t taddr, uint64_t smem_desc) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}\n" ::"r"(taddr), "l"(smem_desc), "r"(pred)
               : "memory");
}

// D[tmem] (+)= A[smem] . B[smem]^T with per-32 block scales from TMEM; one K = 32 step.
__device__ __forceinline__ void tcgen05_mma_mxf8(uint32_t pred, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                                 uint32_t accumulate) {
  asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(pred)
        : "memory");
}

// This thread's TMEM lane (its warp's quarter), 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------- descriptors

// Shared-memory matrix descriptor (tcgen05): start address, leading and stride byte offsets in 16-byte units,
// descriptor version 1 (bits 46-47), swizzle mode in bits 61-63 (0 none, 2 = 128-byte).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout_type & 7u) << 61;
  return d;
}

// Instruction descriptor of kind::mxf8f6f4.block_scale, E4M3 x E4M3 (format 0), both operands K-major, UE8M0
// scales (bit 23), N >> 3 in bits 17-22, M >> 4 in bits 24-28; the byte of the 32-bit scale column each operand
// uses goes into bits 4-5 (B) and 29-30 (A).
__host__ __device__ constexpr uint32_t make_idesc_mxf8(uint32_t m, uint32_t n) {
  return (1u << 23) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ uint32_t idesc_with_sf(uint32_t idesc, uint32_t a_sf_id, uint32_t b_sf_id) {
  return idesc | (b_sf_id << 4) | (a_sf_id << 29);
}

// ---------------------------------------------------------------------------------------------- CTA pairs

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// The shared::cluster address of the same shared-memory offset in the CTA of the given rank.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on an mbarrier anywhere in the cluster (address from map_to_cta). Default semantics (release at CTA
// scope): what travels through these barriers is tensor-memory state ordered by tcgen05 fences, not generic
// memory, and a cluster-scope release would first wait for all of the thread's earlier writes to be visible
// cluster-wide, which costs thousands of cycles behind a stream of output stores.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// A 4-byte store into another CTA's shared memory that completes 4 bytes of a transaction on an mbarrier of that CTA
// (both addresses from map_to_cta): a thread that sees that barrier's phase complete sees the value, as with TMA data.
__device__ __forceinline__ void st_async_u32(uint32_t cluster_addr, uint32_t value, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(cluster_addr), "r"(value), "r"(cluster_bar)
               : "memory");
}

// Tiled loads for a CTA pair: data lands in the issuing CTA's shared memory, the byte count is credited to an
// mbarrier that may live in the pair's other CTA (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t pred, uint32_t smem_dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int32_t x, int32_t y) {
  asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
        "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}\n"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(pred)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d_pair(uint32_t pred, uint32_t smem_dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int32_t c0, int32_t c1, int32_t c2,
                                                 int32_t c3) {
  asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %7, 0;\n\t"
        "@q cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n\t}\n"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3), "r"(pred)
        : "memory");
}

// Tensor memory of both CTAs of a pair: the same warp of each CTA executes these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_out)), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// Completion of the pair's MMAs / copies so far arrives on the mbarrier at this offset in every CTA of cta_mask.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t pred, uint32_t bar_addr, uint16_t cta_mask) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}\n"
               ::"r"(bar_addr), "h"(cta_mask), "r"(pred)
               : "memory");
}

__device__ __forceinline__ void tcgen05_commit_pair(uint32_t pred, uint64_t* bar, uint16_t cta_mask) {
  tcgen05_commit_pair(pred, smem_u32(bar), cta_mask);
}

// Each CTA of the pair copies the scale tile at this offset of its own shared memory into its own TMEM.
__device__ __forceinline__ void tcgen05_cp_32x128b_warpx4_pair(uint32_t pred, uint32_t taddr, uint64_t smem_desc) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n\t}\n" ::"r"(taddr), "l"(smem_desc), "r"(pred)
               : "memory");
}

// One K = 32 step of a 256-row MMA across the pair: each CTA supplies 128 rows of A and half of B's rows from
// the same shared-memory offsets and accumulates its 128 rows of D in its own TMEM.
__device__ __forceinline__ void tcgen05_mma_mxf8_pair(uint32_t pred, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                      uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                                      uint32_t accumulate) {
  asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %7, 0;\n\t"
        "@q tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(pred)
        : "memory");
}

}  // namespace mxb200
