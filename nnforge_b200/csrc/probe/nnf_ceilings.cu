// Memory-system ceilings of the device for the access patterns of the single-launch training batch norm, with no
// arithmetic in the way: a plain copy, a read-only pass, re-reads of a buffer that fits L2, two inputs read and one output
// written without reuse, and the skeleton of the two-read launch itself (statistics items read a channel's planes,
// apply items read them again - from L2 when they follow closely - and write the output; same ticket order, item
// sizes and x[256,256,28,28] layout as the real kernel). Every line: device time per launch by CUDA events, algorithmic
// bytes / time, and that rate against the copy bandwidth given on the command line (default 6537.6 GB/s).
// Stand-alone program: `python bench.py --ceilings` builds nothing, it runs the binary `python -m nnforge_b200.build` made.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <vector>
#include <algorithm>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1); } } while (0)

static double PEAK = 6537.6;

template <class F>
static float timeit(F f, int reps = 20, int warm = 3)
{
	for (int i = 0; i < warm; ++i) f();
	CK(cudaDeviceSynchronize());
	cudaEvent_t e0, e1;
	CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
	CK(cudaEventRecord(e0));
	for (int i = 0; i < reps; ++i) f();
	CK(cudaEventRecord(e1));
	CK(cudaEventSynchronize(e1));
	float ms;
	CK(cudaEventElapsedTime(&ms, e0, e1));
	CK(cudaGetLastError());
	return ms / reps;
}

static void rep(const char * name, float ms, double bytes)
{
	double gbs = bytes / (ms * 1e-3) / 1e9;
	printf("%-84s %8.1f us %8.1f GB/s %6.1f%%\n", name, ms * 1e3, gbs, 100.0 * gbs / PEAK);
	fflush(stdout);
}

// ---- plain kernels ----------------------------------------------------------------------------
template <int L, bool CS>
__global__ void __launch_bounds__(256) copy_kernel(float4 * __restrict__ out, const float4 * __restrict__ in, size_t n4)
{
	const size_t tile = size_t(256) * L;
	for (size_t base = size_t(blockIdx.x) * tile; base < n4; base += size_t(gridDim.x) * tile)
	{
		float4 a[L];
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			size_t i = base + u * 256 + threadIdx.x;
			if (i < n4) a[u] = CS ? __ldcs(in + i) : __ldg(in + i);
		}
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			size_t i = base + u * 256 + threadIdx.x;
			if (i < n4) { if (CS) __stcs(out + i, a[u]); else out[i] = a[u]; }
		}
	}
}

template <int L>
__global__ void __launch_bounds__(256) read_kernel(float * __restrict__ out, const float4 * __restrict__ in, size_t n4, int passes)
{
	const size_t tile = size_t(256) * L;
	float s = 0.f;
	for (int p = 0; p < passes; ++p)
	for (size_t base = size_t(blockIdx.x) * tile; base < n4; base += size_t(gridDim.x) * tile)
	{
		float4 a[L];
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			size_t i = base + u * 256 + threadIdx.x;
			a[u] = make_float4(0, 0, 0, 0);
			if (i < n4) a[u] = __ldg(in + i);
		}
		#pragma unroll
		for (int u = 0; u < L; ++u)
			s += (a[u].x + a[u].y) + (a[u].z + a[u].w);
	}
	if (s == 123.456f) out[0] = s;
}

// two inputs read, one output written (backward-apply pattern, no reuse)
template <int L>
__global__ void __launch_bounds__(256) rrw_kernel(float4 * __restrict__ out, const float4 * __restrict__ a_, const float4 * __restrict__ b_, size_t n4)
{
	const size_t tile = size_t(256) * L;
	for (size_t base = size_t(blockIdx.x) * tile; base < n4; base += size_t(gridDim.x) * tile)
	{
		float4 a[L], b[L];
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			size_t i = base + u * 256 + threadIdx.x;
			if (i < n4) { a[u] = __ldcs(a_ + i); b[u] = __ldcs(b_ + i); }
		}
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			size_t i = base + u * 256 + threadIdx.x;
			if (i < n4) __stcs(out + i, make_float4(a[u].x + b[u].x, a[u].y + b[u].y, a[u].z + b[u].z, a[u].w + b[u].w));
		}
	}
}

// ---- skeleton of the single-launch two-read kernel ----------------------------------------------
// Real layout: x[N][C][196 float4]. S(channel, slice) reads its planes and sums; A(channel, slice)
// reads its planes again (L2) and writes the output. Order: S(chunk 0..lag-1), then S(k+lag), A(k) ...
constexpr uint32_t VPP = 196, NN = 256, CC = 256;
struct skel
{
	const float4 * x; const float4 * dy; float4 * out; float * sink;
	uint32_t * ticket;
	uint32_t es, ea;             // entries per item
	uint32_t split_s, split_a;   // items per channel
	uint32_t chunk;              // channels per chunk
	uint32_t nchunks, lag;
	int policy;                  // 0: S default / A cs; 1: S evict_last
	int fine;                    // interleave S and A items one by one inside a step
	int only;                    // 1: S items only, 2: A items only
};

__device__ __forceinline__ float4 ld_policy(const float4 * p, uint64_t pol)
{
	float4 v;
	asm volatile("ld.global.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(pol));
	return v;
}

template <int L, bool BWD, int MINB>
__global__ void __launch_bounds__(256, MINB) skel_kernel(const skel p)
{
	__shared__ uint32_t s_t;
	if (threadIdx.x == 0) s_t = atomicAdd(p.ticket, 1u);
	__syncthreads();
	uint32_t t = s_t;
	uint32_t apply = 2, ch = 0, sp = 0;
	{
		const uint32_t s_items = p.chunk * p.split_s, a_items = p.chunk * p.split_a;
		uint32_t start = 0;
		for (uint32_t k = 0; k < p.nchunks + p.lag; ++k)
		{
			const bool hs = k < p.nchunks, ha = k >= p.lag;
			if (p.fine && hs && ha)
			{
				const uint32_t items = s_items + a_items;
				if (t - start < items)
				{
					const uint32_t i = t - start;
					const uint32_t sa = (uint64_t(i) * s_items) / items;
					const uint32_t sb = (uint64_t(i + 1) * s_items) / items;
					if (sb > sa) { apply = 0; ch = k * p.chunk + sa / p.split_s; sp = sa % p.split_s; }
					else { const uint32_t j = i - sa; apply = 1; ch = (k - p.lag) * p.chunk + j / p.split_a; sp = j % p.split_a; }
					break;
				}
				start += items;
				continue;
			}
			if (hs)
			{
				if (t - start < s_items) { const uint32_t i = t - start; apply = 0; ch = k * p.chunk + i / p.split_s; sp = i % p.split_s; break; }
				start += s_items;
			}
			if (ha)
			{
				if (t - start < a_items) { const uint32_t i = t - start; apply = 1; ch = (k - p.lag) * p.chunk + i / p.split_a; sp = i % p.split_a; break; }
				start += a_items;
			}
		}
	}
	if (apply > 1) return;
	if (p.only == 1 && apply == 1) return;
	if (p.only == 2 && apply == 0) return;
	const size_t stride = size_t(CC) * VPP;
	if (apply == 0)
	{
		const uint32_t e0 = sp * p.es, e1 = min(e0 + p.es, NN);
		const uint32_t total = (e1 - e0) * VPP;
		const size_t base = size_t(e0) * stride + size_t(ch) * VPP;
		uint64_t pol = 0;
		if (p.policy == 1)
			asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
		float s = 0.f;
		for (uint32_t i0 = threadIdx.x; i0 < total; i0 += 256 * L)
		{
			float4 a[L], d[BWD ? L : 1];
			#pragma unroll
			for (int u = 0; u < L; ++u)
			{
				const uint32_t i = i0 + u * 256;
				a[u] = make_float4(0, 0, 0, 0);
				if (BWD) d[u] = make_float4(0, 0, 0, 0);
				if (i < total)
				{
					const uint32_t lp = i / VPP;
					const size_t off = base + lp * stride + (i - lp * VPP);
					a[u] = p.policy == 1 ? ld_policy(p.x + off, pol) : __ldg(p.x + off);
					if (BWD) d[u] = p.policy == 1 ? ld_policy(p.dy + off, pol) : __ldg(p.dy + off);
				}
			}
			#pragma unroll
			for (int u = 0; u < L; ++u)
			{
				s += (a[u].x + a[u].y) + (a[u].z + a[u].w);
				if (BWD) s += (d[u].x + d[u].y) + (d[u].z + d[u].w);
			}
		}
		if (s == 123.456f) p.sink[0] = s;
		return;
	}
	const uint32_t e0 = sp * p.ea, e1 = min(e0 + p.ea, NN);
	const uint32_t total = (e1 - e0) * VPP;
	const size_t base = size_t(e0) * stride + size_t(ch) * VPP;
	for (uint32_t i0 = threadIdx.x; i0 < total; i0 += 256 * L)
	{
		float4 a[L], d[BWD ? L : 1];
		size_t off[L];
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			const uint32_t i = i0 + u * 256;
			if (i < total)
			{
				const uint32_t lp = i / VPP;
				off[u] = base + lp * stride + (i - lp * VPP);
				a[u] = __ldcs(p.x + off[u]);
				if (BWD) d[u] = __ldcs(p.dy + off[u]);
			}
		}
		#pragma unroll
		for (int u = 0; u < L; ++u)
		{
			const uint32_t i = i0 + u * 256;
			if (i < total)
			{
				float4 o = a[u];
				if (BWD) { o.x += d[u].x; o.y += d[u].y; o.z += d[u].z; o.w += d[u].w; }
				__stcs(p.out + off[u], o);
			}
		}
	}
}

int main(int argc, char ** argv)
{
	if (argc > 1)
		PEAK = atof(argv[1]);
	const size_t E = size_t(256) * 256 * 784;       // elements per tensor
	const size_t n4 = E / 4;
	float * x, * dy, * out, * sink;
	uint32_t * ticket;
	CK(cudaMalloc(&x, E * 4)); CK(cudaMalloc(&dy, E * 4)); CK(cudaMalloc(&out, E * 4)); CK(cudaMalloc(&sink, 1024)); CK(cudaMalloc(&ticket, 1024));
	CK(cudaMemset(x, 0, E * 4)); CK(cudaMemset(dy, 0, E * 4)); CK(cudaMemset(out, 0, E * 4));
	int sms = 0;
	CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
	printf("multiprocessors %d, rates against %.1f GB/s\n", sms, PEAK);
	char name[256];

	// 1. copy
	for (int waves : {1, 4, 32})
	{
		int grid = sms * 8 * waves;
		snprintf(name, sizeof name, "copy 205 MB, L=4, cs, %d waves", waves);
		rep(name, timeit([&] { copy_kernel<4, true><<<grid, 256>>>((float4 *)out, (const float4 *)x, n4); }), 8.0 * E);
	}
	rep("copy 205 MB, L=4, default policy, 32 waves", timeit([&] { copy_kernel<4, false><<<sms * 8 * 32, 256>>>((float4 *)out, (const float4 *)x, n4); }), 8.0 * E);
	rep("copy 205 MB, L=8, cs, 32 waves", timeit([&] { copy_kernel<8, true><<<sms * 8 * 32, 256>>>((float4 *)out, (const float4 *)x, n4); }), 8.0 * E);
	rep("cudaMemcpy D2D 205 MB", timeit([&] { CK(cudaMemcpyAsync(out, x, E * 4, cudaMemcpyDeviceToDevice)); }), 8.0 * E);
	// 2. read only
	for (int waves : {1, 2, 8, 32})
	{
		int grid = sms * 8 * waves;
		snprintf(name, sizeof name, "read-only 205 MB (alternating x, dy), L=4, %d waves", waves);
		int flip = 0;
		rep(name, timeit([&] { read_kernel<4><<<grid, 256>>>(sink, (const float4 *)((flip ^= 1) ? x : dy), n4, 1); }), 4.0 * E);
	}
	{
		int flip = 0;
		rep("read-only 205 MB, L=8, 8 waves", timeit([&] { read_kernel<8><<<sms * 8 * 8, 256>>>(sink, (const float4 *)((flip ^= 1) ? x : dy), n4, 1); }), 4.0 * E);
	}
	// 3. L2-resident reads: buffer of B MB read 16 times inside one launch
	for (int mb : {16, 32, 48, 64, 96})
	{
		size_t b4 = size_t(mb) * 1024 * 1024 / 16;
		snprintf(name, sizeof name, "L2 read: %d MB buffer read 16 times in one launch, L=4", mb);
		rep(name, timeit([&] { read_kernel<4><<<sms * 8, 256>>>(sink, (const float4 *)x, b4, 16); }, 5, 2), 16.0 * mb * 1024 * 1024);
	}
	// 4. read x, dy write dx without reuse
	rep("rrw (x, dy -> dx) 617 MB, L=2, 32 waves", timeit([&] { rrw_kernel<2><<<sms * 8 * 32, 256>>>((float4 *)out, (const float4 *)x, (const float4 *)dy, n4); }), 12.0 * E);
	rep("rrw (x, dy -> dx) 617 MB, L=4, 32 waves", timeit([&] { rrw_kernel<4><<<sms * 8 * 32, 256>>>((float4 *)out, (const float4 *)x, (const float4 *)dy, n4); }), 12.0 * E);

	// 5. skeletons
	auto run_skel = [&](bool bwd, int s_kb, int a_kb, int chunk_mb, int lag, int policy, int fine, int L, int minb, int only = 0)
	{
		skel p = {};
		p.x = (const float4 *)x; p.dy = (const float4 *)dy; p.out = (float4 *)out; p.sink = sink; p.ticket = ticket;
		p.es = std::max(1, s_kb * 1024 / 3136); p.ea = std::max(1, a_kb * 1024 / 3136);
		p.split_s = (NN + p.es - 1) / p.es; p.split_a = (NN + p.ea - 1) / p.ea;
		p.chunk = std::max<uint32_t>(1, uint32_t(double(chunk_mb) * 1024 * 1024 / (256.0 * 3136)));
		while (CC % p.chunk) --p.chunk;
		p.nchunks = CC / p.chunk;
		p.lag = lag;
		p.policy = policy; p.fine = fine; p.only = only;
		uint32_t total = CC * (p.split_s + p.split_a);
		double bytes = double(E) * 4.0 * (only == 1 ? (bwd ? 2 : 1) : (bwd ? 3 : 2));
		auto launch = [&]
		{
			CK(cudaMemsetAsync(ticket, 0, 4));
#define LAUNCH(LL, BB, MM) skel_kernel<LL, BB, MM><<<total, 256>>>(p)
			if (!bwd) { if (L == 4 && minb == 5) LAUNCH(4, false, 5); else if (L == 4 && minb == 8) LAUNCH(4, false, 8); else if (L == 8 && minb == 4) LAUNCH(8, false, 4); else if (L == 2 && minb == 8) LAUNCH(2, false, 8); else { printf("no such variant\n"); exit(1); } }
			else { if (L == 2 && minb == 5) LAUNCH(2, true, 5); else if (L == 2 && minb == 8) LAUNCH(2, true, 8); else if (L == 4 && minb == 4) LAUNCH(4, true, 4); else if (L == 4 && minb == 5) LAUNCH(4, true, 5); else { printf("no such variant\n"); exit(1); } }
		};
		snprintf(name, sizeof name, "skel%s %s S=%dKB A=%dKB chunk=%uch lag=%d policy=%d fine=%d L=%d ctas/SM>=%d", only == 1 ? " S-only" : only == 2 ? " A-only" : "", bwd ? "bwd" : "fwd", s_kb, a_kb, p.chunk, lag, policy, fine, L, minb);
		rep(name, timeit(launch, 10, 3), bytes);
	};
	for (int bwd = 0; bwd < 2; ++bwd)
	{
		const int L0 = bwd ? 2 : 4;
		run_skel(bwd, 48, 64, 16, 1, 0, 0, L0, 5, 1);   // the first read alone
		run_skel(bwd, 48, 64, 16, 1, 0, 0, L0, 5, 2);   // second read + write alone (nothing in L2: every read misses)
		run_skel(bwd, 48, 64, 16, 1, 0, 0, L0, 5);      // both kinds of item, statistics of a chunk then its apply items
		run_skel(bwd, 48, 64, 16, 1, 1, 1, L0, 5);      // first reads marked evict_last, the two kinds interleaved item by item
		run_skel(bwd, 48, 64, 16, 2, 0, 0, L0, 5);      // apply items two chunks behind: the first read has left L2 more often
		run_skel(bwd, 16, 16, 16, 1, 0, 1, L0, 5);      // small items
		run_skel(bwd, 128, 128, 16, 1, 0, 1, L0, 5);    // large items
		run_skel(bwd, 48, 64, 16, 1, 1, 1, bwd ? 4 : 8, 4);   // more loads in flight per thread, fewer CTAs per SM
	}
	printf("done\n");
	return 0;
}
