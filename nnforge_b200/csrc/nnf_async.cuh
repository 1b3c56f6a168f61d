// Thin wrappers over the sm_100a asynchronous-copy instructions used by the single-pass batch-norm
// kernels: mbarriers with bounded waits, bulk copies global -> shared memory (no multicast form is
// used anywhere), and the proxy fence between generic and asynchronous accesses to shared memory.
#pragma once

#include "nnf_common.cuh"

namespace nnf
{
	constexpr uint32_t kWaitLimit = 1u << 26; // try_wait rounds before giving up (each suspends up to ~1 us)

	__device__ __forceinline__ uint32_t smem_addr(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }

	__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count)
	{
		asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_addr(bar)), "r"(count));
	}

	__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, uint32_t bytes)
	{
		asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_addr(bar)), "r"(bytes) : "memory");
	}

	__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity)
	{
		uint32_t ok;
		asm volatile(
			"{\n"
			".reg .pred p;\n"
			"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
			"selp.u32 %0, 1, 0, p;\n"
			"}\n" : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
		return ok != 0;
	}

	// Bounded wait; returns false when the limit ran out.
	__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity)
	{
		for (uint32_t i = 0; i < kWaitLimit; ++i)
			if (mbar_try_wait(bar, parity))
				return true;
		return false;
	}

	// global -> this CTA's shared memory, `bytes` a multiple of 16, both addresses 16-byte aligned
	__device__ __forceinline__ void bulk_load(void * dst_smem, const void * src_gmem, uint32_t bytes, uint64_t * bar)
	{
		asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
			:: "r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)) : "memory");
	}

	__device__ __forceinline__ void fence_proxy_async()
	{
		asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
	}
}
