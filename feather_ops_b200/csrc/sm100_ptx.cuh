// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM allocation,
// UMMA issue/commit, TMEM loads) and the shared-memory / instruction descriptors the UMMA unit reads.
//
// Every wait in here is bounded. A wait that runs out records where it gave up in a global status word,
// raises a CTA-wide abort flag and returns false, so the kernel can drain and exit with the context intact.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace feather {

// ---------------------------------------------------------------------------------------------------------
// Status word (one 2 x u32 record per launch, owned by the host side). 0 = clean.
// ---------------------------------------------------------------------------------------------------------
enum WaitSite : uint32_t {
    kSiteNone = 0,
    kSiteLoadEmpty = 1,   // TMA producer waiting for a free load slot
    kSiteLoadFull = 2,    // consumer waiting for TMA bytes
    kSiteOperandEmpty = 3,  // operand producer waiting for the MMA to release a converted-operand slot
    kSiteOperandFull = 4,   // MMA issuer waiting for the converted operand
    kSiteTmemEmpty = 5,   // MMA issuer waiting for the epilogue to drain an accumulator
    kSiteTmemFull = 6,    // epilogue waiting for the accumulator
    kSiteStore = 7,       // epilogue waiting for its bulk stores
};

// Roughly two seconds at the maximum SM clock. A healthy kernel never waits more than a few tile times.
constexpr long long kWaitLimitCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Per-CTA view of the launch's status record plus the CTA-wide abort flag in shared memory.
struct WaitGuard {
    volatile uint32_t* abort_flag;  // shared memory, one word per CTA
    uint32_t* status;               // global memory, two words: [0] = site | (tag << 8), [1] = blockIdx.x

    __device__ __forceinline__ bool aborted() const { return *abort_flag != 0u; }

    __device__ __noinline__ void give_up(uint32_t site, uint32_t tag) const {
        *abort_flag = 1u;
        if (atomicCAS(status, 0u, site | (tag << 8)) == 0u) {
            status[1] = blockIdx.x;
        }
        __threadfence();
    }

    // Wait for the phase with `parity` to complete. False means the CTA is aborting (this wait ran out,
    // or another one did): the caller must stop touching the pipeline and fall through to the teardown.
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, uint32_t site, uint32_t tag = 0) const {
        return wait_at_most(bar, parity, site, tag, kWaitLimitCycles);
    }

    // The same wait with the limit given by the caller (the kernels use `wait`; the self-test passes a short limit).
    __device__ __forceinline__ bool wait_at_most(uint64_t* bar, uint32_t parity, uint32_t site, uint32_t tag, long long limit_cycles) const {
        if (mbar_try_wait(bar, parity)) return true;
        const long long start = clock64();
        uint32_t polls = 0;
        while (true) {
            if (mbar_try_wait(bar, parity)) return true;
            if ((++polls & 0x3fu) == 0u) {
                if (aborted()) return false;
                if (clock64() - start > limit_cycles) {
                    give_up(site, tag);
                    return false;
                }
            }
        }
    }
};

// Programmatic dependent launch. A kernel launched with the programmatic-stream-serialization attribute may start while the
// kernel before it in the stream is still running; `grid_dependency_wait` returns once that kernel has completed and its
// memory is visible (at once when the launch carries no such attribute). `grid_launch_dependents` tells the scheduler that
// the kernel after this one may start as soon as every CTA of this one has called it or exited.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Generic-proxy writes to shared memory (st.shared) -> visible to the async proxy (UMMA, TMA stores).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------------------
// Per-thread asynchronous copies (cp.async, generic proxy)
// ---------------------------------------------------------------------------------------------------------
// 4 bytes global -> shared. `live == false` writes zeros without reading `src` (which must still be a
// valid address).
__device__ __forceinline__ void cp_async_4(uint32_t smem_dst, const void* src, bool live) {
    const uint32_t src_bytes = live ? 4u : 0u;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// TMA loads / stores (never with cluster multicast)
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// Tensor memory
// ---------------------------------------------------------------------------------------------------------
// One full warp. `columns` is a power of two in [32, 512]. The base address lands in `*smem_slot`.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(columns) : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// mbarrier arrive once every UMMA issued so far by this thread has finished reading its operands
// and writing its accumulator.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16/bf16 operands, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], int8 operands, int32 accumulate.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread `lane` of the warp gets row (lane) of its lane quarter.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// CTA pairs (cluster of two, tcgen05 cta_group::2). The UMMA is issued by the even CTA of the pair and
// reads A rows and B columns from both CTAs' shared memory at the same offsets; each CTA's tensor memory
// receives its own 128 accumulator rows. Nothing here uses a multicast qualifier: barriers in the
// peer CTA are signalled one by one through their shared::cluster addresses.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

// 16 bytes into another CTA's shared memory (distributed shared memory; the address comes from map_to_cta)
__device__ __forceinline__ void st_shared_cluster_v4(uint32_t cluster_addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// Arrive on a barrier given by its shared::cluster address (this CTA's or the peer's). Plain release
// semantics: a cluster-scope release here costs over a thousand cycles per arrive and is not needed,
// the operand data is published to the async proxy by the fence that precedes the arrive.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(columns) : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// arrive (once the pair's UMMAs issued so far have completed) on the barrier at `cluster_addr`
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------------------------------------
// Instruction descriptor fields (32 bit): [4,6) accumulator format, [7,10) A format, [10,13) B format,
// [15] A major, [16] B major (0 = K-major), [17,23) N >> 3, [24,29) M >> 4.
constexpr uint32_t kFmtF16 = 0;   // kind::f16 operand formats
constexpr uint32_t kFmtBF16 = 1;
constexpr uint32_t kFmtU8 = 0;    // kind::i8 operand formats
constexpr uint32_t kFmtS8 = 1;
constexpr uint32_t kAccF32 = 1;
constexpr uint32_t kAccS32 = 2;

__host__ __device__ constexpr uint32_t make_idesc(uint32_t acc_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
    return (acc_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Shared-memory matrix descriptor (64 bit): [0,14) address >> 4, [16,30) leading byte offset >> 4,
// [32,46) stride byte offset >> 4, [46,48) = 1 (descriptor version of this architecture),
// [61,64) swizzle mode (0 none, 2 = 128 B).
constexpr uint64_t kSwizzleNone = 0;
constexpr uint64_t kSwizzle128B = 2;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swizzle) {
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}

// K-major operand tile whose rows are exactly one 128-byte swizzle span (64 halfwords or 128 bytes of K):
// 8-row groups are 1024 bytes apart, the leading offset is unused by the hardware for this mode.
// Stepping along K inside the span is a plain start-address bump (the XOR pattern is applied on address
// bits that the bump does not touch as long as the tile base is 1024-byte aligned).
__device__ __forceinline__ uint64_t make_desc_sw128_kmajor(uint32_t smem_addr) {
    return make_smem_desc(smem_addr, 16u, 1024u, kSwizzle128B);
}

// MN-major operand tile of one 128-byte swizzle span along M or N (128 bytes of 8-bit elements) and any number of
// contraction rows: a row is the span for one contraction index, 8-row groups are 1024 bytes apart (the stride offset);
// the leading offset would separate spans along M / N and is unused with a single one. Stepping along the contraction
// is a start-address bump of whole 8-row groups. The instruction descriptor must carry the matching major bit.
__device__ __forceinline__ uint64_t make_desc_sw128_mnmajor(uint32_t smem_addr) {
    return make_smem_desc(smem_addr, 16u, 1024u, kSwizzle128B);
}
constexpr uint32_t kIdescBMajorMN = 1u << 16;

// Tile walk of the persistent pair kernels: row tiles fastest inside a band of `band` row tiles, all column tiles
// of a band before the next band. The activation rows of one band (sized by the host to a few tens of MB) then stay
// in L2 while the band sweeps the weight; with row tiles fastest over the whole matrix, a tall activation matrix
// would be re-read from HBM once per column tile.
__device__ __forceinline__ void banded_tile(int tile, int tiles_m, int tiles_n, int band, int& tile_m, int& tile_n) {
    const int per_band = band * tiles_n;
    const int b = tile / per_band;
    const int r = tile - b * per_band;
    const int left = tiles_m - b * band;
    const int rows_here = left < band ? left : band;
    tile_n = r / rows_here;
    tile_m = b * band + (r - tile_n * rows_here);
}

// Position of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128B-swizzled tile: same mapping as
// a TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace feather
