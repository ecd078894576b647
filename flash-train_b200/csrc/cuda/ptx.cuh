// Inline-PTX building blocks for sm_100a: mbarriers with bounded waits, TMA
// tile loads, tcgen05 (tensor memory allocation, MMA issue, commit, loads) and
// the proxy / tcgen05 fences that order them.
//
// Every wait is bounded: a wait that does not complete within kWaitBudgetNs
// returns false, and callers then raise the kernel's abort flag, stop issuing
// work and leave through the normal exit path (which frees tensor memory).
// Nothing here traps or spins forever.
#ifndef FTCUDA_PTX_CUH_
#define FTCUDA_PTX_CUH_

#include <cstdint>

namespace ftcuda {

// Upper bound for one wait. Legitimate waits in these kernels last
// microseconds; two seconds only ever elapses when a peer role has stopped.
constexpr unsigned long long kWaitBudgetNs = 2000000000ULL;

__device__ __forceinline__ std::uint32_t smemAddress(const void* pointer) {
    return static_cast<std::uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ unsigned long long globalTimerNs() {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    return now;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbarrierInit(std::uint64_t* barrier, std::uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddress(barrier)), "r"(arrivals));
}

// Makes freshly initialised barriers visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fenceBarrierInit() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbarrierArrive(std::uint64_t* barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddress(barrier)) : "memory");
}

__device__ __forceinline__ void mbarrierArriveExpectTx(std::uint64_t* barrier, std::uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddress(barrier)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbarrierTryWait(std::uint64_t* barrier, std::uint32_t parity) {
    std::uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(smemAddress(barrier)), "r"(parity)
        : "memory");
    return done != 0;
}

// Non-blocking test of the same condition (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbarrierTestWait(std::uint64_t* barrier, std::uint32_t parity) {
    std::uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(smemAddress(barrier)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity to complete. Gives up -- returning
// false -- when *abort_flag becomes nonzero or `budget_ns` has elapsed.
__device__ __forceinline__ bool mbarrierWaitFor(std::uint64_t* barrier, std::uint32_t parity,
                                                const volatile int* abort_flag, unsigned long long budget_ns) {
    if (mbarrierTryWait(barrier, parity)) { return true; }
    const unsigned long long start = globalTimerNs();
    std::uint32_t spins            = 0;
    while (true) {
        if (mbarrierTryWait(barrier, parity)) { return true; }
        if ((++spins & 0xFF) == 0) {
            if (*abort_flag != 0) { return false; }
            if (globalTimerNs() - start > budget_ns) { return false; }
        }
    }
}

// The same with the kernels' budget.
__device__ __forceinline__ bool mbarrierWait(std::uint64_t* barrier, std::uint32_t parity,
                                             const volatile int* abort_flag) {
    return mbarrierWaitFor(barrier, parity, abort_flag, kWaitBudgetNs);
}

// ---------------------------------------------------------------- programmatic dependent launch

// Blocks the calling thread until the grids this grid depends on (the kernels before it in the
// stream) have completed and their memory operations are visible. Returns at once when the grid was
// launched without programmatic stream serialization. Every thread that touches global memory
// calls it first; what precedes it (barrier setup, tensor-memory allocation) overlaps the
// predecessor's tail.
__device__ __forceinline__ void gridDependencyWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Lets the next grid in the stream (if it was launched with programmatic stream serialization)
// start its CTAs as soon as every CTA of this grid has got here or exited. The dependent's own
// gridDependencyWait still holds it back until this grid has completed.
__device__ __forceinline__ void gridDependencyLaunchDependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- fences

// Orders this thread's generic-proxy shared-memory writes before later
// async-proxy reads (tcgen05.mma operand fetch, TMA stores).
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tcgen05FenceBeforeSync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05FenceAfterSync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA

// 2-D tiled load global -> shared, completion counted in bytes on `barrier`.
// `x` is the innermost (contiguous) coordinate; x * 4 bytes must be a multiple
// of 16 (callers only pass multiples of 32 elements).
__device__ __forceinline__ void tmaLoad2d(void* smem_destination, const void* tensor_map, std::uint64_t* barrier,
                                          std::int32_t x, std::int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smemAddress(smem_destination)),
        "l"(reinterpret_cast<std::uint64_t>(tensor_map)), "r"(smemAddress(barrier)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void prefetchTensorMap(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<std::uint64_t>(tensor_map)) : "memory");
}

// ---------------------------------------------------------------- tcgen05

// Whole-warp calls. `columns` is a power of two in [32, 512]. The base address
// of the allocation is written to *result_in_smem.
__device__ __forceinline__ void tmemAllocate(std::uint32_t* result_in_smem, std::uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddress(result_in_smem)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmemFree(std::uint32_t base, std::uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// Shared-memory operand descriptor for a K-major tile stored as rows of 128
// bytes with the 128-byte swizzle (exactly what a TMA load with
// CU_TENSOR_MAP_SWIZZLE_128B produces; the tile base must be 1024-byte aligned).
// Eight consecutive rows form one 1024-byte swizzle atom, so the stride between
// 8-row groups is 1024 bytes; the leading-dimension offset is unused for this
// layout. Bits: [0,14) address>>4, [32,46) stride>>4, [46,48) version = 1,
// [61,64) layout = 2 (128-byte swizzle).
__device__ __forceinline__ std::uint64_t umaDescriptorK128(std::uint32_t smem_address) {
    std::uint64_t descriptor = 0;
    descriptor |= static_cast<std::uint64_t>((smem_address & 0x3FFFF) >> 4);
    descriptor |= static_cast<std::uint64_t>(1024 >> 4) << 32;
    descriptor |= static_cast<std::uint64_t>(1) << 46;
    descriptor |= static_cast<std::uint64_t>(2) << 61;
    return descriptor;
}

// Shared-memory operand descriptor for an MN-major tile (the M or N index is
// the contiguous one) of 32-bit elements. The only layout the tensor cores take
// for such an operand is the 128-byte swizzle with a 32-byte base: rows of 128
// bytes hold 32 consecutive MN elements at one k, their 32-byte quarters XOR-ed
// with k % 4; four consecutive k form one 512-byte swizzle atom. (A TMA load
// with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B of a box 32 (MN) x 4j (K) produces j
// such atoms 512 bytes apart.) `mn_atom_bytes` is the distance between atoms
// along MN (the next 32 elements; "leading" offset, bits [16,30)),
// `k_atom_bytes` the distance between atoms along K (the next 4 k; "stride"
// offset, bits [32,46)). Layout code 1 in bits [61,64).
__device__ __forceinline__ std::uint64_t umaDescriptorMn128Base32(std::uint32_t smem_address, std::uint32_t mn_atom_bytes,
                                                                  std::uint32_t k_atom_bytes) {
    std::uint64_t descriptor = 0;
    descriptor |= static_cast<std::uint64_t>((smem_address & 0x3FFFF) >> 4);
    descriptor |= static_cast<std::uint64_t>((mn_atom_bytes >> 4) & 0x3FFF) << 16;
    descriptor |= static_cast<std::uint64_t>((k_atom_bytes >> 4) & 0x3FFF) << 32;
    descriptor |= static_cast<std::uint64_t>(1) << 46;
    descriptor |= static_cast<std::uint64_t>(1) << 61;
    return descriptor;
}

// Bit of the instruction descriptor that declares the B operand MN-major.
constexpr std::uint32_t kUmaBMnMajor = 1u << 16;

// Instruction descriptor for kind::tf32, FP32 accumulation, both operands
// K-major, dense. Bits: [4,6) D format (1 = F32), [7,10) A format (2 = TF32),
// [10,13) B format (2 = TF32), 15/16 A/B major (0 = K), [17,23) N>>3,
// [24,29) M>>4.
__host__ __device__ constexpr std::uint32_t umaInstructionTf32(std::uint32_t m, std::uint32_t n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread. accumulate == 0
// overwrites D.
__device__ __forceinline__ void umaTf32(std::uint32_t d_tmem, std::uint64_t a_descriptor, std::uint64_t b_descriptor,
                                        std::uint32_t instruction, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_descriptor), "l"(b_descriptor), "r"(instruction), "r"(accumulate)
        : "memory");
}

// Same with the A operand in tensor memory: M rows in lanes 0..M-1, the 8 K
// elements of this instruction in 8 consecutive 32-bit columns at a_tmem.
__device__ __forceinline__ void umaTf32TmemA(std::uint32_t d_tmem, std::uint32_t a_tmem, std::uint64_t b_descriptor,
                                             std::uint32_t instruction, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_descriptor), "r"(instruction), "r"(accumulate)
        : "memory");
}

// Arrives once on `barrier` when every MMA this thread issued so far has
// finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umaCommit(std::uint64_t* barrier) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smemAddress(barrier))
                 : "memory");
}

// ---------------------------------------------------------------- thread-block clusters

__device__ __forceinline__ std::uint32_t clusterCtaRank() {
    std::uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
__device__ __forceinline__ void clusterBarrierArrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void clusterBarrierWait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Whole-warp load of 32 lanes x 32 consecutive 32-bit columns: thread t of the
// warp receives lane (lane_base + t), columns [column, column + 32). The wait
// for the load sits in the same asm statement so that no use of the registers
// can be scheduled before it.
__device__ __forceinline__ void tmemLoad32(std::uint32_t address, float (&out)[32]) {
    std::uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) { out[i] = __uint_as_float(r[i]); }
}

// Three such loads (96 consecutive columns) under one wait: the round trip to tensor memory is
// paid once for the whole strip.
__device__ __forceinline__ void tmemLoad96(std::uint32_t address, float (&out)[96]) {
    std::uint32_t r[96];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%96];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%97];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, "
        "%80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95}, [%98];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]),
          "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]),
          "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]),
          "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]),
          "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95])
        : "r"(address), "r"(address + 32), "r"(address + 64)
        : "memory");
#pragma unroll
    for (int i = 0; i < 96; ++i) { out[i] = __uint_as_float(r[i]); }
}

// setmaxnreg: a warpgroup (warps 4i .. 4i+3, every warp with the same count) gives registers back
// to the CTA's pool or takes some from it; counts are multiples of 8.
template<int kRegisters>
__device__ __forceinline__ void registersShrink() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegisters));
}
template<int kRegisters>
__device__ __forceinline__ void registersGrow() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegisters));
}

// Same for 16 consecutive columns.
__device__ __forceinline__ void tmemLoad16(std::uint32_t address, float (&out)[16]) {
    std::uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) { out[i] = __uint_as_float(r[i]); }
}

// Whole-warp store of 32 lanes x 16 consecutive columns, completed before return.
__device__ __forceinline__ void tmemStore16(std::uint32_t address, const float (&in)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n\t"
        "tcgen05.wait::st.sync.aligned;" ::"r"(address),
        "r"(__float_as_uint(in[0])), "r"(__float_as_uint(in[1])), "r"(__float_as_uint(in[2])),
        "r"(__float_as_uint(in[3])), "r"(__float_as_uint(in[4])), "r"(__float_as_uint(in[5])),
        "r"(__float_as_uint(in[6])), "r"(__float_as_uint(in[7])), "r"(__float_as_uint(in[8])),
        "r"(__float_as_uint(in[9])), "r"(__float_as_uint(in[10])), "r"(__float_as_uint(in[11])),
        "r"(__float_as_uint(in[12])), "r"(__float_as_uint(in[13])), "r"(__float_as_uint(in[14])),
        "r"(__float_as_uint(in[15]))
        : "memory");
}

// The same store without waiting for it; tmemStoreWait() completes all of a
// thread's earlier tensor-memory stores.
__device__ __forceinline__ void tmemStore16NoWait(std::uint32_t address, const float (&in)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(address),
        "r"(__float_as_uint(in[0])), "r"(__float_as_uint(in[1])), "r"(__float_as_uint(in[2])),
        "r"(__float_as_uint(in[3])), "r"(__float_as_uint(in[4])), "r"(__float_as_uint(in[5])),
        "r"(__float_as_uint(in[6])), "r"(__float_as_uint(in[7])), "r"(__float_as_uint(in[8])),
        "r"(__float_as_uint(in[9])), "r"(__float_as_uint(in[10])), "r"(__float_as_uint(in[11])),
        "r"(__float_as_uint(in[12])), "r"(__float_as_uint(in[13])), "r"(__float_as_uint(in[14])),
        "r"(__float_as_uint(in[15]))
        : "memory");
}

__device__ __forceinline__ void tmemStoreWait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

}  // namespace ftcuda

#endif
