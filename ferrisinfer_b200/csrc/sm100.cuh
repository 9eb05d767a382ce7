// Blackwell (sm_100a) primitives in inline PTX: mbarriers with bounded waits, TMA tiled loads,
// tcgen05 (tensor memory, MMA, commit, load), ldmatrix / mma.sync helpers, and the host side of
// tensor maps.  Every wait has an iteration limit: when it runs out the kernel records where it
// gave up in a device status word (read by ferris_kernel_status()) and carries on to its exit
// path, so a fault in a pipeline shows as an error code, never as a hang.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---------------------------------------------------------------------------------------------
// status word
// ---------------------------------------------------------------------------------------------
// 0 = fine.  Otherwise (code << 16) | detail; codes below.
#define FERRIS_STATUS_MBAR_TIMEOUT 1
#define FERRIS_STATUS_BAD_INDEX 2

// Device address of the status word of the current device (host function; kernels get it as an argument).
int* ferris_status_ptr();

__device__ __forceinline__ void ferris_report(int* status, int code, int detail) {
    if (status) atomicCAS(status, 0, (code << 16) | (detail & 0xffff));
}

// ---------------------------------------------------------------------------------------------
// shared-memory addresses, mbarriers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    // make the initialised barriers visible to the async proxy (TMA, tcgen05.commit)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for the phase of `parity` to complete.  Returns false (and records `where`) if it does not
// within the limit: about a second of polling, far beyond any legitimate wait of these kernels.
#ifndef FERRIS_WAIT_LIMIT
#define FERRIS_WAIT_LIMIT (1u << 24)
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int where) {
    for (uint32_t i = 0; i < FERRIS_WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    ferris_report(status, FERRIS_STATUS_MBAR_TIMEOUT, where);
    return false;
}

// ---------------------------------------------------------------------------------------------
// thread-block clusters: rank, barrier over all threads of all CTAs, loads from a peer's shared memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The fp32 at shared address `addr` (this CTA's numbering) in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ float ld_peer_shared_f32(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Four consecutive fp32 at shared address `addr` (16-byte aligned) in the shared memory of CTA `rank`.
__device__ __forceinline__ float4 ld_peer_shared_f32x4(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(remote)
                 : "memory");
    return v;
}

// The barrier in two halves, for every thread on its own (no warp has to be converged): a thread arrives once and
// waits once per phase, in that order.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }

// Stores an fp32 at shared address `addr` (this CTA's numbering) in the shared memory of CTA `rank` of the cluster.
// The target CTA must be running (a cluster barrier that it has arrived on says so), and sees the value after the
// next cluster barrier with release / acquire.
__device__ __forceinline__ void st_peer_shared_f32(uint32_t addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// TMA: tiled 2-D load global -> shared, completion on an mbarrier.  No multicast.
// The innermost coordinate x times the element size must be a multiple of 16 bytes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// The same with three coordinates (x innermost).
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// TMA tile shared -> global: a plain store, or an element-wise add into global memory (done by the memory
// system, so the old values are never read by the SM).  Completion is tracked per thread in bulk groups.
// Coordinates must not be negative; rows and columns beyond the tensor's extent are dropped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's bulk groups have finished READING shared memory (the source may be rewritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all of this thread's bulk groups are complete (their writes are done)
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Byte offset of (row, 16-byte chunk) inside a tile that TMA wrote with 128-byte swizzle
// (rows of 128 bytes, tile base aligned to 1024 bytes).
__device__ __forceinline__ uint32_t swizzle128(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// ---------------------------------------------------------------------------------------------
// warp-level matrix helpers (mma.sync m16n8k16 bf16 -> fp32, ldmatrix)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// The 8 x 8 matrix of 16-bit values that the warp holds one row pair per thread (row lane / 4, columns 2 (lane % 4)
// and the next), transposed: the same thread then holds the same place of the transposed matrix.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory and the 5th-generation MMA
// ---------------------------------------------------------------------------------------------
// One warp allocates `cols` columns (a power of two >= 32) and writes the TMEM address to *dst (shared).
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulation; issued by ONE thread.
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The mbarrier gets one arrival when all tcgen05 operations issued so far by this thread are done.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&r)[32]) {
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

// 32 lanes x 64 consecutive fp32 columns.
__device__ __forceinline__ void tmem_load_32x64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
          "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
          "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
          "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
          "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_load_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile written by TMA with 128-byte swizzle:
// rows of 64 bf16 (128 bytes), groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address
    d |= (uint64_t)1 << 16;                              // leading byte offset: unused with swizzle, 1 by convention
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                              // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}

// The same for an MN-major operand (rows of the tile run along K, as TMA writes a [K rows x 64 columns] box): groups of
// 8 K rows 1024 bytes apart; column groups of 64 (when the operand is wider than 64) `mn_group_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn_major_sw128(uint32_t smem_addr, uint32_t mn_group_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address
    d |= (uint64_t)((mn_group_bytes >> 4) & 0x3FFF) << 16;  // leading byte offset: between column groups of 64
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset: 8 K rows x 128 bytes
    d |= (uint64_t)1 << 46;                              // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, tile M x N.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4)                 // D is fp32
           | (1u << 7)               // A is bf16
           | (1u << 10)              // B is bf16
           | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// CTA pairs (cta_group::2): two CTAs of a cluster with ranks 2i and 2i + 1 run ONE MMA of 256 rows, 128 per
// CTA, with each CTA holding its own A rows and one half of the B rows in its shared memory, and each CTA's
// half of the accumulator in its own tensor memory.  The even CTA (the leader) issues the MMAs; both CTAs load
// with TMA and signal the LEADER's mbarrier; tcgen05.commit arrives on a barrier at the same offset in both.
// ---------------------------------------------------------------------------------------------
// The shared::cluster address of this CTA's shared address `addr` in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}

// One arrival on an mbarrier given by its shared::cluster address (own or a peer's).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA tile load into THIS CTA's shared memory whose bytes count on the mbarrier at `bar_cluster_addr` (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

// Tensor memory for a pair: the same warp of BOTH CTAs calls this with the same `dst` offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem of both CTAs] (+)= A * B^T over the pair: 256 rows (128 from each CTA's A tile), N columns (each CTA holds
// N / 2 rows of B).  Issued by ONE thread of the leader CTA; the descriptors are the leader's (same offsets in the peer).
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                      uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One arrival on the mbarrier at `bar`'s offset in every CTA of `cta_mask` (bit r = CTA rank r of the cluster) when all
// MMAs issued so far by this thread are done.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(cta_mask)
                 : "memory");
}

// ---------------------------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------------------------
// A 2-D bf16 tensor [rows, cols] with `row_stride` elements between rows, read in boxes of
// box_rows x box_cols with 128-byte swizzle (box_cols * 2 bytes must be 128).
// Returns 0 or a negative error (text in ferris_last_error()).
int ferris_make_tensor_map_planes(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t plane_bytes,
                                  uint32_t box_rows);
int ferris_make_tensor_map_kblocks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                                   uint32_t box_rows, uint32_t box_kblocks);
int ferris_make_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                              uint32_t box_rows, uint32_t box_cols);

// The same for an fp32 tensor (boxes of box_rows x 32 floats = 128 bytes, 128-byte swizzle): the target of
// TMA stores and TMA add-reductions of output tiles.
int ferris_make_tensor_map_2d_f32(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                                  uint64_t row_stride, uint32_t box_rows);
