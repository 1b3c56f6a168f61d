// Single-pass training batch norm (+ activation chain) for one GPU: every element of x (and dy) is
// read from HBM once and every output written once - 8 bytes/element forward, 12 backward - where the
// two-kernel form (nnf_bn_train.cu) moves 12 and 20.
//
// A thread-block CLUSTER owns one channel at a time. The channel's slab (N planes of H*W floats) is
// split over the cluster's CTAs, each CTA pulls its planes into shared memory with bulk async copies
// (cp.async.bulk global -> shared, completion on an mbarrier), reduces its part with warp shuffles,
// and the CTAs exchange their partial sums through distributed shared memory (st.shared::cluster +
// barrier.cluster). With the statistics known, every CTA normalises its planes straight out of
// shared memory and streams the result to HBM with 128-bit stores.
//
// The kernels run only when a channel's slab fits the shared memory of one cluster; otherwise the
// entry points fall back to the two-kernel form. They are single-GPU kernels: a batch-sharded run
// needs the all-reduce between statistics and normalisation and uses the two-kernel form.
//
// Waiting: the only spin is the mbarrier wait for this CTA's own bulk copies; it is bounded, and on
// expiry the kernel raises an error word and carries on (results are then invalid, nothing hangs).
#include "nnf_common.cuh"
#include "nnf_async.cuh"

#include <mutex>
#include <stdlib.h>

namespace nnf
{
	namespace
	{
		constexpr int kMaxCluster = 16;

		__device__ __forceinline__ uint32_t cluster_rank()
		{
			uint32_t r;
			asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
			return r;
		}

		__device__ __forceinline__ void cluster_sync_all()
		{
			asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
		}

		// store a double into the same shared-memory variable of CTA `rank` of this cluster
		__device__ __forceinline__ void dsmem_store(double * local_ptr, uint32_t rank, double v)
		{
			uint32_t remote;
			asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local_ptr)), "r"(rank));
			asm volatile("st.shared::cluster.f64 [%0], %1;" :: "r"(remote), "d"(v) : "memory");
		}

		__device__ __forceinline__ double warp_sum_d(double v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			return v;
		}

		__device__ __forceinline__ unsigned long long global_timer()
		{
			unsigned long long t;
			asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
			return t;
		}

		struct fused_params
		{
			const float * x;
			const float * dy;        // backward only
			float * out;             // y (forward) or dx (backward)
			const float * gamma;
			const float * beta;
			float * saved;           // forward: written {mean, invstd}; backward: read
			float * sums;            // forward: {sum x, sum x^2} (may be null); backward: bsums[3C] written
			float * grad_gamma, * grad_beta, * grad_mean, * grad_invsigma, * grad_slope;
			const float * mean, * invsigma;
			float entry_count;
			int add;
			act_chain chain;
			uint32_t n, c, hw;
			uint32_t planes_per_cta;
			uint32_t cluster;        // CTAs per cluster
			uint32_t nbuf;           // slab buffers per CTA (2: the next channel loads while this one is processed)
			uint32_t slab_floats;    // floats per slab buffer
			fastdiv d_vpp;           // float4 per plane
			double count;            // elements per channel
			float eps;
			int * error;             // raised when a bounded wait ran out
			unsigned long long * trace; // tuning aid (normally null): per CTA and iteration, 5 globaltimer stamps
			uint32_t stagger_ns;     // odd clusters start this much later, so that clusters run out of phase
		};

		// Clusters that all start together stay in lockstep (every channel costs the same), so HBM sees
		// alternating bursts of loads and stores with idle gaps in between. Delaying every other cluster by
		// about half an iteration keeps the two halves out of phase for the whole kernel.
		__device__ __forceinline__ void stagger_start(uint32_t cluster_id, uint32_t ns)
		{
			if ((cluster_id & 1) && ns)
			{
				const unsigned long long t0 = global_timer();
				for (int i = 0; i < 4096 && global_timer() - t0 < ns; ++i)
					__nanosleep(200);
			}
		}

		// Block-wide sums in double; every thread returns with the totals (through shared memory).
		template <int K>
		__device__ __forceinline__ void block_sum_all(double (&v)[K], double * s_red)
		{
			const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
			#pragma unroll
			for (int k = 0; k < K; ++k)
				v[k] = warp_sum_d(v[k]);
			if (lane == 0)
			{
				#pragma unroll
				for (int k = 0; k < K; ++k)
					s_red[w * K + k] = v[k];
			}
			__syncthreads();
			#pragma unroll
			for (int k = 0; k < K; ++k)
			{
				double t = 0.0;
				for (int i = 0; i < nw; ++i)
					t += s_red[i * K + k];
				v[k] = t;
			}
		}

		// ---- forward ---------------------------------------------------------------------------
		template <int A0, int A1>
		__global__ void __launch_bounds__(1024, 1) bn_train_fwd_cluster_kernel(const fused_params p)
		{
			extern __shared__ __align__(128) unsigned char s_dyn[];
			float * slab_base = reinterpret_cast<float *>(s_dyn);
			__shared__ __align__(8) uint64_t s_bar[2];
			__shared__ double s_red[32 * 2];  // one slot per warp (up to 32 warps)
			__shared__ double s_exch[2][kMaxCluster][2];

			const uint32_t rank = cluster_rank();
			const uint32_t cluster_id = blockIdx.x / p.cluster;
			const uint32_t nclusters = gridDim.x / p.cluster;
			const uint32_t e0 = rank * p.planes_per_cta;
			const uint32_t e1 = min(e0 + p.planes_per_cta, p.n);
			const uint32_t np = e1 > e0 ? e1 - e0 : 0;
			const uint32_t plane_bytes = p.hw * 4;
			const uint32_t vpp = p.hw >> 2;
			const uint32_t nvec = np * vpp;

			if (threadIdx.x == 0)
			{
				mbar_init(&s_bar[0], 1);
				mbar_init(&s_bar[1], 1);
				asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
			}
			__syncthreads();

			// pulls this CTA's planes of channel ch into slab buffer b (executed by warp 0)
			auto issue_load = [&](uint32_t ch, uint32_t b)
			{
				if (threadIdx.x == 0)
				{
					fence_proxy_async(); // earlier generic reads of the buffer are ordered before the async writes
					mbar_expect_tx(&s_bar[b], np * plane_bytes);
				}
				__syncwarp();
				float * dst = slab_base + size_t(b) * p.slab_floats;
				for (uint32_t pl = threadIdx.x; pl < np; pl += 32)
					bulk_load(dst + size_t(pl) * p.hw, p.x + (size_t(e0 + pl) * p.c + ch) * p.hw, plane_bytes, &s_bar[b]);
			};

			stagger_start(cluster_id, p.stagger_ns);
			if (threadIdx.x < 32 && cluster_id < p.c)
				issue_load(cluster_id, 0);

			uint32_t it = 0;
			for (uint32_t ch = cluster_id; ch < p.c; ch += nclusters, ++it)
			{
				// 1. buffer and barrier phase of this channel; start the next channel's load
				const uint32_t b = p.nbuf == 2 ? (it & 1) : 0;
				const uint32_t parity = p.nbuf == 2 ? ((it >> 1) & 1) : (it & 1);
				if (threadIdx.x < 32)
				{
					if (p.nbuf == 2)
					{
						if (ch + nclusters < p.c)
							issue_load(ch + nclusters, b ^ 1); // that buffer was released by the barrier ending the previous iteration
					}
					else if (it > 0)
						issue_load(ch, 0);
				}
				unsigned long long * tr = (p.trace && threadIdx.x == 0 && it < 32) ? p.trace + (size_t(blockIdx.x) * 32 + it) * 5 : nullptr;
				if (tr) tr[0] = global_timer();
				const float * slab = slab_base + size_t(b) * p.slab_floats;
				const float gamma = __ldg(p.gamma + ch), beta = __ldg(p.beta + ch);
				const float slope = chain_slope(p.chain, ch);
				if (!mbar_wait(&s_bar[b], parity) && p.error)
					*p.error = 1;

				if (tr) tr[1] = global_timer();
				// 2. partial sums of this CTA
				float s = 0.0F, q = 0.0F;
				const float4 * slab4 = reinterpret_cast<const float4 *>(slab);
				for (uint32_t i = threadIdx.x; i < nvec; i += blockDim.x)
				{
					const float4 a = slab4[i];
					s += (a.x + a.y) + (a.z + a.w);
					q += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w);
				}
				double acc[2] = {double(s), double(q)};
				block_sum_all<2>(acc, s_red);

				if (tr) tr[2] = global_timer();
				// 3. exchange through distributed shared memory, double-buffered by iteration parity
				const uint32_t buf = it & 1;
				if (threadIdx.x < p.cluster)
				{
					dsmem_store(&s_exch[buf][rank][0], threadIdx.x, acc[0]);
					dsmem_store(&s_exch[buf][rank][1], threadIdx.x, acc[1]);
				}
				__syncwarp();
				cluster_sync_all();
				if (tr) tr[3] = global_timer();
				double ts = 0.0, tq = 0.0;
				for (uint32_t r = 0; r < p.cluster; ++r)
				{
					ts += s_exch[buf][r][0];
					tq += s_exch[buf][r][1];
				}
				const double m = ts / p.count;
				double var = tq / p.count - m * m;
				var = var < 0.0 ? 0.0 : var;
				const float mean = float(m);
				const float invstd = float(1.0 / sqrt(var + double(p.eps)));
				if (rank == 0 && threadIdx.x == 0)
				{
					if (p.saved)
					{
						p.saved[ch] = mean;
						p.saved[p.c + ch] = invstd;
					}
					if (p.sums)
					{
						p.sums[ch] = float(ts);
						p.sums[p.c + ch] = float(tq);
					}
				}
				const float mult = __fmul_rn(gamma, invstd);
				const float add = __fsub_rn(beta, __fmul_rn(mult, mean));

				// 4. normalise + activations out of shared memory, stream to HBM
				for (uint32_t i = threadIdx.x; i < nvec; i += blockDim.x)
				{
					const uint32_t pl = p.d_vpp.div(i);
					const uint32_t v = i - pl * vpp;
					const float4 a = slab4[i];
					float4 o;
					o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.x, mult), add), slope);
					o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.y, mult), add), slope);
					o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.z, mult), add), slope);
					o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.w, mult), add), slope);
					st_stream(reinterpret_cast<float4 *>(p.out + (size_t(e0 + pl) * p.c + ch) * p.hw) + v, o);
				}
				__syncthreads(); // this buffer is free again
				if (tr) tr[4] = global_timer();
			}
		}

		// ---- backward -------------------------------------------------------------------------
		// Shared memory holds du (the gradient that reaches the batch-norm output) for this CTA's planes.
		// Pass 1 streams x and dy from HBM once, recomputes the activation chain once, stores du and
		// accumulates {sum du, sum du*xhat, sum dslope}; after the cluster exchange pass 2 reads du from
		// shared memory and x again - a few microseconds after its first read, so from L2 - and streams dx.
		template <int A0, int A1>
		__global__ void __launch_bounds__(512, 2) bn_train_bwd_cluster_kernel(const fused_params p)
		{
			extern __shared__ __align__(128) unsigned char s_dyn[];
			float4 * slab4 = reinterpret_cast<float4 *>(s_dyn);
			__shared__ double s_red[16 * 3];
			__shared__ double s_exch[2][kMaxCluster][3];

			const uint32_t rank = cluster_rank();
			const uint32_t cluster_id = blockIdx.x / p.cluster;
			const uint32_t nclusters = gridDim.x / p.cluster;
			const uint32_t e0 = rank * p.planes_per_cta;
			const uint32_t e1 = min(e0 + p.planes_per_cta, p.n);
			const uint32_t np = e1 > e0 ? e1 - e0 : 0;
			const uint32_t vpp = p.hw >> 2;
			const uint32_t nvec = np * vpp;
			constexpr int kU = 2;
			stagger_start(cluster_id, p.stagger_ns);

			uint32_t it = 0;
			for (uint32_t ch = cluster_id; ch < p.c; ch += nclusters, ++it)
			{
				unsigned long long * tr = (p.trace && threadIdx.x == 0 && it < 32) ? p.trace + (size_t(blockIdx.x) * 32 + it) * 5 : nullptr;
				if (tr) tr[0] = global_timer();
				const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
				const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
				const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
				const float slope = chain_slope(p.chain, ch);
				const size_t chan_off = size_t(ch) * p.hw;
				const size_t entry_stride = size_t(p.c) * p.hw;

				// pass 1
				float sb = 0.0F, sg = 0.0F, ss = 0.0F;
				auto element = [&](float x, float dy) -> float
				{
					const float u = __fadd_rn(__fmul_rn(x, mult), add);
					float term;
					const float du = chain_backward<A0, A1>(p.chain, u, dy, slope, term);
					const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
					sb += du;
					sg += du * xhat;
					ss += term;
					return du;
				};
				for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kU)
				{
					float4 a[kU], d[kU];
					#pragma unroll
					for (int u = 0; u < kU; ++u)
					{
						const uint32_t i = i0 + u * blockDim.x;
						if (i < nvec)
						{
							const uint32_t pl = p.d_vpp.div(i);
							const size_t off = size_t(e0 + pl) * entry_stride + chan_off + size_t(i - pl * vpp) * 4;
							a[u] = __ldg(reinterpret_cast<const float4 *>(p.x + off));      // stays in L2 for pass 2
							d[u] = ld_stream(reinterpret_cast<const float4 *>(p.dy + off));
						}
					}
					#pragma unroll
					for (int u = 0; u < kU; ++u)
					{
						const uint32_t i = i0 + u * blockDim.x;
						if (i < nvec)
							slab4[i] = make_float4(element(a[u].x, d[u].x), element(a[u].y, d[u].y), element(a[u].z, d[u].z), element(a[u].w, d[u].w));
					}
				}
				if (tr) tr[1] = global_timer();
				double acc[3] = {double(sb), double(sg), double(ss)};
				block_sum_all<3>(acc, s_red);
				if (tr) tr[2] = global_timer();

				// exchange through distributed shared memory, double-buffered by iteration parity
				const uint32_t buf = it & 1;
				if (threadIdx.x < p.cluster)
				{
					dsmem_store(&s_exch[buf][rank][0], threadIdx.x, acc[0]);
					dsmem_store(&s_exch[buf][rank][1], threadIdx.x, acc[1]);
					dsmem_store(&s_exch[buf][rank][2], threadIdx.x, acc[2]);
				}
				__syncwarp();
				cluster_sync_all();
				if (tr) tr[3] = global_timer();
				double tb = 0.0, tg = 0.0, tsl = 0.0;
				for (uint32_t r = 0; r < p.cluster; ++r)
				{
					tb += s_exch[buf][r][0];
					tg += s_exch[buf][r][1];
					tsl += s_exch[buf][r][2];
				}
				const float fb = float(tb), fg = float(tg), fs = float(tsl);
				if (rank == 0 && threadIdx.x == 0)
				{
					if (p.sums)
					{
						p.sums[ch] = fb;
						p.sums[p.c + ch] = fg;
						p.sums[2 * p.c + ch] = fs;
					}
					// per-channel gradients accumulate (batch_norm_layer_updater_cuda.cu:138-139, 167-182)
					if (p.grad_beta) p.grad_beta[ch] += fb;
					if (p.grad_gamma) p.grad_gamma[ch] += fg;
					if (p.grad_slope) p.grad_slope[ch] += fs;
					if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (mean - p.mean[ch]);
					if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (invstd - p.invsigma[ch]);
				}
				// the same float-rounded sums the two-kernel form passes between its kernels
				const float c2 = float(double(fb) / p.count);
				const float c3 = float(double(fg) / p.count);

				// pass 2
				for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kU)
				{
					float4 a[kU], o[kU];
					size_t pos[kU];
					#pragma unroll
					for (int u = 0; u < kU; ++u)
					{
						const uint32_t i = i0 + u * blockDim.x;
						o[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						if (i < nvec)
						{
							const uint32_t pl = p.d_vpp.div(i);
							pos[u] = size_t(e0 + pl) * entry_stride + chan_off + size_t(i - pl * vpp) * 4;
							a[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + pos[u]));
							if (p.add)
								o[u] = ld_stream(reinterpret_cast<const float4 *>(p.out + pos[u]));
						}
					}
					#pragma unroll
					for (int u = 0; u < kU; ++u)
					{
						const uint32_t i = i0 + u * blockDim.x;
						if (i < nvec)
						{
							const float4 du = slab4[i];
							auto dx_of = [&](float x, float g, float old) -> float
							{
								const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
								const float r = mult * ((g - c2) - xhat * c3);
								return p.add ? old + r : r;
							};
							st_stream(reinterpret_cast<float4 *>(p.out + pos[u]),
								make_float4(dx_of(a[u].x, du.x, o[u].x), dx_of(a[u].y, du.y, o[u].y), dx_of(a[u].z, du.z, o[u].z), dx_of(a[u].w, du.w, o[u].w)));
						}
					}
				}
				__syncthreads(); // du of this channel is consumed; the slab may be overwritten
				if (tr) tr[4] = global_timer();
			}
		}

		// ---- variants that keep the slab in L2 instead of shared memory ------------------------------
		// One cluster per channel, launched for all channels at once. Pass 1 streams this CTA's planes from
		// HBM (default cache policy, so the lines stay in L2) and reduces; the cluster exchanges its partial
		// sums; pass 2 reads the same planes again a few microseconds later - from L2 - and streams the
		// result out with evict-first stores. No shared-memory slab, so any N and H*W fit; the number of
		// channels in flight (and with it the L2 footprint) is bounded by a shared-memory reservation that
		// limits how many CTAs an SM holds.
#ifndef NNF_L2_THREADS
#define NNF_L2_THREADS 512
#endif
#ifndef NNF_L2_MIN_CTAS
#define NNF_L2_MIN_CTAS 3
#endif
#ifndef NNF_L2_UNROLL
#define NNF_L2_UNROLL 2
#endif
		constexpr int kL2Threads = NNF_L2_THREADS;
		constexpr int kL2MinCtas = NNF_L2_MIN_CTAS;

		template <int A0, int A1>
		__global__ void __launch_bounds__(kL2Threads, kL2MinCtas) bn_train_fwd_l2_kernel(const fused_params p)
		{
			__shared__ double s_red[32 * 2];
			__shared__ double s_exch[kMaxCluster][2];
			const uint32_t rank = cluster_rank();
			const uint32_t ch = blockIdx.x / p.cluster;
			const uint32_t e0 = rank * p.planes_per_cta;
			const uint32_t e1 = min(e0 + p.planes_per_cta, p.n);
			const uint32_t np = e1 > e0 ? e1 - e0 : 0;
			const uint32_t vpp = p.hw >> 2;
			const uint32_t nvec = np * vpp;
			const size_t entry_stride = size_t(p.c) * p.hw;
			const size_t base = size_t(e0) * entry_stride + size_t(ch) * p.hw;
			constexpr int kU = NNF_L2_UNROLL;

			float s = 0.0F, q = 0.0F;
			for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kU)
			{
				float4 a[kU];
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					const uint32_t i = i0 + u * blockDim.x;
					a[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					if (i < nvec)
					{
						const uint32_t pl = p.d_vpp.div(i);
						a[u] = __ldg(reinterpret_cast<const float4 *>(p.x + base + pl * entry_stride) + (i - pl * vpp));
					}
				}
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					s += (a[u].x + a[u].y) + (a[u].z + a[u].w);
					q += (a[u].x * a[u].x + a[u].y * a[u].y) + (a[u].z * a[u].z + a[u].w * a[u].w);
				}
			}
			double acc[2] = {double(s), double(q)};
			block_sum_all<2>(acc, s_red);
			if (threadIdx.x < p.cluster)
			{
				dsmem_store(&s_exch[rank][0], threadIdx.x, acc[0]);
				dsmem_store(&s_exch[rank][1], threadIdx.x, acc[1]);
			}
			__syncwarp();
			cluster_sync_all();
			double ts = 0.0, tq = 0.0;
			for (uint32_t r = 0; r < p.cluster; ++r)
			{
				ts += s_exch[r][0];
				tq += s_exch[r][1];
			}
			const double m = ts / p.count;
			double var = tq / p.count - m * m;
			var = var < 0.0 ? 0.0 : var;
			const float mean = float(m);
			const float invstd = float(1.0 / sqrt(var + double(p.eps)));
			if (rank == 0 && threadIdx.x == 0)
			{
				if (p.saved)
				{
					p.saved[ch] = mean;
					p.saved[p.c + ch] = invstd;
				}
				if (p.sums)
				{
					p.sums[ch] = float(ts);
					p.sums[p.c + ch] = float(tq);
				}
			}
			const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
			const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			const float slope = chain_slope(p.chain, ch);

			for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kU)
			{
				float4 a[kU];
				size_t pos[kU];
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					const uint32_t i = i0 + u * blockDim.x;
					if (i < nvec)
					{
						const uint32_t pl = p.d_vpp.div(i);
						pos[u] = base + pl * entry_stride + size_t(i - pl * vpp) * 4;
						a[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + pos[u])); // last use: evict first
					}
				}
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					const uint32_t i = i0 + u * blockDim.x;
					if (i < nvec)
					{
						float4 o;
						o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].x, mult), add), slope);
						o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].y, mult), add), slope);
						o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].z, mult), add), slope);
						o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].w, mult), add), slope);
						st_stream(reinterpret_cast<float4 *>(p.out + pos[u]), o);
					}
				}
			}
		}

		template <int A0, int A1>
		__global__ void __launch_bounds__(kL2Threads, kL2MinCtas) bn_train_bwd_l2_kernel(const fused_params p)
		{
			__shared__ double s_red[32 * 3];
			__shared__ double s_exch[kMaxCluster][3];
			const uint32_t rank = cluster_rank();
			const uint32_t ch = blockIdx.x / p.cluster;
			const uint32_t e0 = rank * p.planes_per_cta;
			const uint32_t e1 = min(e0 + p.planes_per_cta, p.n);
			const uint32_t np = e1 > e0 ? e1 - e0 : 0;
			const uint32_t vpp = p.hw >> 2;
			const uint32_t nvec = np * vpp;
			const size_t entry_stride = size_t(p.c) * p.hw;
			const size_t base = size_t(e0) * entry_stride + size_t(ch) * p.hw;
			constexpr int kU = 2;

			const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
			const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
			const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			const float slope = chain_slope(p.chain, ch);

			float sb = 0.0F, sg = 0.0F, ss = 0.0F;
			auto du_of = [&](float x, float dy, float& term) -> float
			{
				const float u = __fadd_rn(__fmul_rn(x, mult), add);
				return chain_backward<A0, A1>(p.chain, u, dy, slope, term);
			};
			for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kU)
			{
				float4 a[kU], d[kU];
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					const uint32_t i = i0 + u * blockDim.x;
					if (i < nvec)
					{
						const uint32_t pl = p.d_vpp.div(i);
						const size_t pos = base + pl * entry_stride + size_t(i - pl * vpp) * 4;
						a[u] = __ldg(reinterpret_cast<const float4 *>(p.x + pos));
						d[u] = __ldg(reinterpret_cast<const float4 *>(p.dy + pos));
					}
				}
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					if (i0 + u * blockDim.x < nvec)
					{
						const float xs[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
						const float ds[4] = {d[u].x, d[u].y, d[u].z, d[u].w};
						#pragma unroll
						for (int k = 0; k < 4; ++k)
						{
							float term;
							const float du = du_of(xs[k], ds[k], term);
							const float xhat = __fmul_rn(__fsub_rn(xs[k], mean), invstd);
							sb += du;
							sg += du * xhat;
							ss += term;
						}
					}
				}
			}
			double acc[3] = {double(sb), double(sg), double(ss)};
			block_sum_all<3>(acc, s_red);
			if (threadIdx.x < p.cluster)
			{
				dsmem_store(&s_exch[rank][0], threadIdx.x, acc[0]);
				dsmem_store(&s_exch[rank][1], threadIdx.x, acc[1]);
				dsmem_store(&s_exch[rank][2], threadIdx.x, acc[2]);
			}
			__syncwarp();
			cluster_sync_all();
			double tb = 0.0, tg = 0.0, tsl = 0.0;
			for (uint32_t r = 0; r < p.cluster; ++r)
			{
				tb += s_exch[r][0];
				tg += s_exch[r][1];
				tsl += s_exch[r][2];
			}
			const float fb = float(tb), fg = float(tg), fs = float(tsl);
			if (rank == 0 && threadIdx.x == 0)
			{
				if (p.sums)
				{
					p.sums[ch] = fb;
					p.sums[p.c + ch] = fg;
					p.sums[2 * p.c + ch] = fs;
				}
				if (p.grad_beta) p.grad_beta[ch] += fb;
				if (p.grad_gamma) p.grad_gamma[ch] += fg;
				if (p.grad_slope) p.grad_slope[ch] += fs;
				if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (mean - p.mean[ch]);
				if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (invstd - p.invsigma[ch]);
			}
			const float c2 = float(double(fb) / p.count);
			const float c3 = float(double(fg) / p.count);

			for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += blockDim.x * kU)
			{
				float4 a[kU], d[kU], o[kU];
				size_t pos[kU];
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					const uint32_t i = i0 + u * blockDim.x;
					o[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					if (i < nvec)
					{
						const uint32_t pl = p.d_vpp.div(i);
						pos[u] = base + pl * entry_stride + size_t(i - pl * vpp) * 4;
						a[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + pos[u]));
						d[u] = ld_stream(reinterpret_cast<const float4 *>(p.dy + pos[u]));
						if (p.add)
							o[u] = ld_stream(reinterpret_cast<const float4 *>(p.out + pos[u]));
					}
				}
				#pragma unroll
				for (int u = 0; u < kU; ++u)
				{
					if (i0 + u * blockDim.x < nvec)
					{
						auto dx_of = [&](float x, float dy, float old) -> float
						{
							float term;
							const float du = du_of(x, dy, term);
							const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
							const float r = mult * ((du - c2) - xhat * c3);
							return p.add ? old + r : r;
						};
						st_stream(reinterpret_cast<float4 *>(p.out + pos[u]),
							make_float4(dx_of(a[u].x, d[u].x, o[u].x), dx_of(a[u].y, d[u].y, o[u].y), dx_of(a[u].z, d[u].z, o[u].z), dx_of(a[u].w, d[u].w, o[u].w)));
					}
				}
			}
		}

		// ---- host side ---------------------------------------------------------------------------
		struct fused_plan
		{
			int cluster;
			int threads;
			int grid;            // CTAs (multiple of cluster)
			size_t smem;
			uint32_t planes_per_cta;
			int nbuf;
		};

		int * error_word();

		template <class Kernel>
		bool plan_fused(fused_plan& plan, Kernel kernel, int64_t n, int64_t c, int64_t hw, int tensors, bool single_buffer_only = false, int max_threads = 1024)
		{
			if (hw % 4 != 0 || n < 1)
				return false;
			const size_t plane_bytes = size_t(hw) * 4 * tensors;
			const size_t smem_cap = 220 * 1024;
			// first choice: two single-buffered CTAs per SM (the phases of two channels overlap, and small
			// CTAs let more clusters fit the GPCs: 33 clusters of 8 against 15 with one 200 KB CTA per SM);
			// then one CTA per SM with two slab buffers; then one single-buffered CTA per SM
			static const int kClusters[] = {8, 4, 2, 1, 16};
			static const size_t kBudget[] = {108 * 1024, smem_cap, smem_cap};
			static const int kBufs[] = {1, 2, 1};
			static const int kThreadsPerCta[] = {512, 1024, 1024};
			const char * forced = getenv("NNF_FUSED_CLUSTER"); // tuning aids: force a cluster size / buffer count
			const char * forced_buf = getenv("NNF_FUSED_NBUF");
			for (int choice = 0; choice < 3; ++choice)
				for (int cl : kClusters)
				{
					const size_t budget = kBudget[choice];
					const int nbuf = kBufs[choice];
					if (cl > n || (forced && atoi(forced) != cl) || (forced_buf && atoi(forced_buf) != nbuf) || (single_buffer_only && nbuf != 1))
						continue;
					const uint32_t ppc = (uint32_t)div_up(n, cl);
					const size_t smem = size_t(ppc) * plane_bytes * nbuf;
					if (smem > budget || size_t(ppc) * hw * 4 >= (size_t(1) << 20))
						continue;
					if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
					{
						cudaGetLastError();
						continue;
					}
					if (cl > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
					{
						cudaGetLastError();
						continue;
					}
					cudaLaunchConfig_t cfg = {};
					cudaLaunchAttribute attr;
					attr.id = cudaLaunchAttributeClusterDimension;
					attr.val.clusterDim.x = cl; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
					cfg.gridDim = dim3(cl, 1, 1);
					cfg.blockDim = dim3(kThreadsPerCta[choice] < max_threads ? kThreadsPerCta[choice] : max_threads, 1, 1);
					cfg.dynamicSmemBytes = smem;
					cfg.attrs = &attr;
					cfg.numAttrs = 1;
					int max_clusters = 0;
					if (cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg) != cudaSuccess || max_clusters < 1)
					{
						cudaGetLastError();
						continue;
					}
					int clusters = max_clusters < c ? max_clusters : (int)c;
					// even out the rounds: ceil(c / clusters) rounds need no more than that many clusters
					const int rounds = (int)div_up(c, clusters);
					clusters = (int)div_up(c, rounds);
					plan.cluster = cl;
					plan.threads = kThreadsPerCta[choice] < max_threads ? kThreadsPerCta[choice] : max_threads;
					plan.grid = clusters * cl;
					plan.smem = smem;
					plan.planes_per_cta = ppc;
					plan.nbuf = nbuf;
					if (getenv("NNF_FUSED_VERBOSE"))
						fprintf(stderr, "nnf fused plan: cluster %d, %d buffer(s), %zu B smem, %d clusters of max %d\n", cl, nbuf, smem, clusters, max_clusters);
					return true;
				}
			return false;
		}

		template <class Kernel>
		int launch_fused(Kernel kernel, const fused_plan& plan, const fused_params& p, cudaStream_t s, const char * what)
		{
			cudaLaunchConfig_t cfg = {};
			cudaLaunchAttribute attr;
			attr.id = cudaLaunchAttributeClusterDimension;
			attr.val.clusterDim.x = plan.cluster; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
			cfg.gridDim = dim3(plan.grid, 1, 1);
			cfg.blockDim = dim3(plan.threads, 1, 1);
			cfg.dynamicSmemBytes = plan.smem;
			cfg.stream = s;
			cfg.attrs = &attr;
			cfg.numAttrs = 1;
			cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
			return NNF_OK;
		}
	}
}

namespace nnf
{
	namespace
	{
		// Launch shape of the L2-resident variants: cluster size, planes per CTA, and the shared-memory
		// reservation that keeps the channels in flight (clusters resident at once x slab bytes) under
		// the L2 budget.
		struct l2_plan
		{
			int cluster;
			uint32_t planes_per_cta;
			size_t reserve_smem;
		};

		bool plan_l2(l2_plan& plan, int64_t n, int64_t c, int64_t hw, int tensors)
		{
			if (hw % 4 != 0 || n < 1)
				return false;
			int cl = 8;
			while (cl > 1 && cl > n)
				cl >>= 1;
			const char * forced = getenv("NNF_L2_CLUSTER"); // tuning aid
			if (forced && atoi(forced) >= 1 && atoi(forced) <= 8)
				cl = atoi(forced);
			const double slab = double(n) * double(hw) * 4.0 * tensors;
			const double budget = (getenv("NNF_L2_BUDGET_MB") ? atof(getenv("NNF_L2_BUDGET_MB")) : 64.0) * 1024.0 * 1024.0;
			// channels in flight = SMs * CTAs per SM / cluster size
			int ctas_per_sm = int(budget / (slab * double(kSmCount) / cl));
			if (ctas_per_sm < 1)
				return false; // even one CTA per SM would overflow the budget: use the two-kernel form
			const int max_ctas = 2048 / kL2Threads;
			if (ctas_per_sm >= max_ctas)
				ctas_per_sm = max_ctas;
			plan.cluster = cl;
			plan.planes_per_cta = (uint32_t)div_up(n, cl);
			plan.reserve_smem = ctas_per_sm >= max_ctas ? 0 : size_t(225 * 1024) / ctas_per_sm - 2048;
			return true;
		}

		template <class Kernel>
		int launch_l2(Kernel kernel, const l2_plan& plan, const fused_params& p, cudaStream_t s, const char * what)
		{
			cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(plan.reserve_smem > 48 * 1024 ? plan.reserve_smem : 48 * 1024));
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
			cudaLaunchConfig_t cfg = {};
			cudaLaunchAttribute attr;
			attr.id = cudaLaunchAttributeClusterDimension;
			attr.val.clusterDim.x = plan.cluster; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
			cfg.gridDim = dim3(p.c * plan.cluster, 1, 1);
			cfg.blockDim = dim3(kL2Threads, 1, 1);
			cfg.dynamicSmemBytes = plan.reserve_smem;
			cfg.stream = s;
			cfg.attrs = &attr;
			cfg.numAttrs = 1;
			e = cudaLaunchKernelEx(&cfg, kernel, p);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
			return NNF_OK;
		}

		// Which form the single-GPU entry points use (NNF_FUSED_MODE, a tuning aid):
		//   0 (default)  single launch of statistics and apply items, second read from L2 (nnf_bn_chain.cu);
		//                shapes it does not take fall through to mode 3
		//   1            L2-resident cluster kernels for both directions
		//   2            shared-memory slab cluster kernels for both directions
		//   3            forward: shared-memory slab cluster kernel; backward: the two-kernel form
		// Measured on B200, x[256,256,28,28], PReLU+ELU: forward 95 us (single launch) / 98 us (slab) / 108 us
		// (L2 clusters) / 110 us (two kernels); backward 154-160 us (single launch) / 185 us (slab) / 172-192 us
		// (L2 clusters) / 176-183 us (two kernels). The slab kernels move only 8 / 12 bytes per element through
		// HBM (ncu: x and dy read once) but are bound by what an SM keeps in flight; the forms that read twice
		// run at the rate at which the SMs can exchange data with L2, whether or not the second read hits.
		int fused_mode()
		{
			const char * m = getenv("NNF_FUSED_MODE");
			return m ? atoi(m) : 0;
		}
	}
}

// Error word of the cluster kernels: a device variable inside the library, so that reaching it needs
// no allocation (the enqueue path never allocates).
static __device__ int nnf_fused_error_word;

namespace nnf
{
	namespace
	{
		int * error_word()
		{
			static std::mutex mu;
			static int * words[64] = {};
			int dev = 0;
			if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
				return nullptr;
			std::lock_guard<std::mutex> lock(mu);
			if (!words[dev])
			{
				int * w = nullptr;
				if (cudaGetSymbolAddress((void **)&w, nnf_fused_error_word) != cudaSuccess)
				{
					cudaGetLastError();
					return nullptr;
				}
				words[dev] = w;
			}
			return words[dev];
		}
	}
}

namespace nnf
{
	// the same error word, for the other translation units that have bounded waits
	int * device_error_word() { return error_word(); }
}

using namespace nnf;

extern "C" int nnf_bn_train_fwd(nnf_stream_t stream, float * y, float * saved, float * sums, const float * x,
	const float * gamma, const float * beta, float eps,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes)
{
	if (n <= 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_fwd: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (!y || !x || !gamma || !beta || !saved)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_fwd: null pointer");
	act_chain chain;
	int st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	const int k0 = chain.n > 0 ? chain.a[0].kind : NNF_ACT_NONE;
	const int k1 = chain.n > 1 ? chain.a[1].kind : NNF_ACT_NONE;
	typedef void (*kernel_t)(const fused_params);
	kernel_t kernel = bn_train_fwd_cluster_kernel<-1, 0>;
	if (chain.n == 0)
		kernel = bn_train_fwd_cluster_kernel<NNF_ACT_NONE, 0>;
	else if (k0 == NNF_ACT_PRELU && k1 == NNF_ACT_ELU)
		kernel = bn_train_fwd_cluster_kernel<NNF_ACT_PRELU, NNF_ACT_ELU>;
	else if (k0 == NNF_ACT_RELU && k1 == NNF_ACT_NONE)
		kernel = bn_train_fwd_cluster_kernel<NNF_ACT_RELU, 0>;

	const bool shape_ok = n <= 0x7fffffff && c <= 0x7fffffff / 8 && hw <= 0x7fffffff && n * hw < (int64_t(1) << 31) && aligned16(x) && aligned16(y);
	if (fused_mode() == 0 && shape_ok)
	{
		st = chain_forward_launch((cudaStream_t)stream, y, saved, sums, x, gamma, beta, eps, chain, n, c, hw, workspace, workspace_bytes);
		if (st != 1)
			return st;
	}
	l2_plan lp;
	if (fused_mode() == 1 && shape_ok && plan_l2(lp, n, c, hw, 1))
	{
		kernel_t k2 = bn_train_fwd_l2_kernel<-1, 0>;
		if (chain.n == 0)
			k2 = bn_train_fwd_l2_kernel<NNF_ACT_NONE, 0>;
		else if (k0 == NNF_ACT_PRELU && k1 == NNF_ACT_ELU)
			k2 = bn_train_fwd_l2_kernel<NNF_ACT_PRELU, NNF_ACT_ELU>;
		else if (k0 == NNF_ACT_RELU && k1 == NNF_ACT_NONE)
			k2 = bn_train_fwd_l2_kernel<NNF_ACT_RELU, 0>;
		fused_params q = {};
		q.x = x; q.out = y; q.gamma = gamma; q.beta = beta; q.saved = saved; q.sums = sums;
		q.chain = chain;
		q.n = (uint32_t)n; q.c = (uint32_t)c; q.hw = (uint32_t)hw;
		q.planes_per_cta = lp.planes_per_cta;
		q.cluster = (uint32_t)lp.cluster;
		q.d_vpp = fastdiv((uint32_t)(hw / 4));
		q.count = double(n) * double(hw);
		q.eps = eps;
		return launch_l2(k2, lp, q, (cudaStream_t)stream, "bn_train_fwd_l2_kernel");
	}
	fused_plan plan;
	const bool fits = shape_ok && plan_fused(plan, kernel, n, c, hw, 1);
	if (!fits)
	{
		// two-kernel form
		float * tmp_sums = sums;
		if (!tmp_sums)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_fwd: this shape needs the two-kernel form, which requires the sums buffer");
		st = nnf_bn_train_stats(stream, tmp_sums, x, n, c, hw, workspace, workspace_bytes);
		if (st != NNF_OK)
			return st;
		return nnf_bn_train_apply_act(stream, y, saved, x, gamma, beta, tmp_sums, double(n) * double(hw), eps, acts, n_acts, n, c, hw);
	}
	fused_params p = {};
	p.x = x; p.out = y; p.gamma = gamma; p.beta = beta; p.saved = saved; p.sums = sums;
	p.chain = chain;
	p.n = (uint32_t)n; p.c = (uint32_t)c; p.hw = (uint32_t)hw;
	p.planes_per_cta = plan.planes_per_cta;
	p.cluster = (uint32_t)plan.cluster;
	p.nbuf = (uint32_t)plan.nbuf;
	p.slab_floats = (uint32_t)(plan.planes_per_cta * hw);
	p.d_vpp = fastdiv((uint32_t)(hw / 4));
	p.count = double(n) * double(hw);
	p.eps = eps;
	p.error = error_word();
	p.stagger_ns = getenv("NNF_FUSED_STAGGER_NS") ? (uint32_t)atoi(getenv("NNF_FUSED_STAGGER_NS")) : 0;
	{
		const char * t = getenv("NNF_FUSED_TRACE"); // tuning aid: address of a device buffer, as a decimal number
		p.trace = t ? reinterpret_cast<unsigned long long *>(strtoull(t, nullptr, 10)) : nullptr;
	}
	return launch_fused(kernel, plan, p, (cudaStream_t)stream, "bn_train_fwd_cluster_kernel");
}

// Reads and clears the error word that the cluster kernels raise when a bounded wait runs out.
// Synchronises the device; meant for tests and debugging, not for the enqueue path.
extern "C" int nnf_fused_error_check(void)
{
	int * w = error_word();
	if (!w)
		return 0;
	int v = 0;
	if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
		return -1;
	if (v)
		cudaMemset(w, 0, sizeof(int));
	return v;
}

extern "C" int nnf_bn_train_bwd(nnf_stream_t stream, float * dx, float * bsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination,
	void * workspace, size_t workspace_bytes)
{
	if (n <= 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (!dx || !dy || !x || !gamma || !beta || !saved || !bsums)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd: null pointer");
	if ((grad_mean && !mean) || (grad_invsigma && !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd: running-statistics gradients requested without the running statistics");
	act_chain chain;
	int st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	chain_fill_backward_constants(chain, acts, n_acts);
	int prelus = 0;
	for (int i = 0; i < chain.n; ++i)
		prelus += chain.a[i].kind == NNF_ACT_PRELU;
	if (prelus > 1)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_bwd: at most one PReLU per fused chain");
	typedef void (*kernel_t)(const fused_params);
	kernel_t kernel = bn_train_bwd_cluster_kernel<-1, 0>;
	switch (chain_id(chain))
	{
	case 0: kernel = bn_train_bwd_cluster_kernel<NNF_ACT_NONE, 0>; break;
	case 1: kernel = bn_train_bwd_cluster_kernel<NNF_ACT_PRELU, NNF_ACT_ELU>; break;
	case 2: kernel = bn_train_bwd_cluster_kernel<NNF_ACT_RELU, 0>; break;
	default: break;
	}
	const bool shape_ok = n <= 0x7fffffff && c <= 0x7fffffff / 8 && hw <= 0x7fffffff && n * hw < (int64_t(1) << 31) && aligned16(x) && aligned16(dy) && aligned16(dx);
	if (fused_mode() == 0 && shape_ok && !add_to_destination)
	{
		st = chain_backward_launch((cudaStream_t)stream, dx, bsums, dy, x, gamma, beta, saved, chain, grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope,
			mean, invsigma, entry_count, n, c, hw, workspace, workspace_bytes);
		if (st != 1)
			return st;
	}
	l2_plan lp;
	if (fused_mode() == 1 && shape_ok && plan_l2(lp, n, c, hw, 2))
	{
		kernel_t k2 = bn_train_bwd_l2_kernel<-1, 0>;
		switch (chain_id(chain))
		{
		case 0: k2 = bn_train_bwd_l2_kernel<NNF_ACT_NONE, 0>; break;
		case 1: k2 = bn_train_bwd_l2_kernel<NNF_ACT_PRELU, NNF_ACT_ELU>; break;
		case 2: k2 = bn_train_bwd_l2_kernel<NNF_ACT_RELU, 0>; break;
		default: break;
		}
		fused_params q = {};
		q.x = x; q.dy = dy; q.out = dx; q.gamma = gamma; q.beta = beta; q.saved = const_cast<float *>(saved); q.sums = bsums;
		q.grad_gamma = grad_gamma; q.grad_beta = grad_beta; q.grad_mean = grad_mean; q.grad_invsigma = grad_invsigma; q.grad_slope = grad_slope;
		q.mean = mean; q.invsigma = invsigma; q.entry_count = entry_count;
		q.add = add_to_destination ? 1 : 0;
		q.chain = chain;
		q.n = (uint32_t)n; q.c = (uint32_t)c; q.hw = (uint32_t)hw;
		q.planes_per_cta = lp.planes_per_cta;
		q.cluster = (uint32_t)lp.cluster;
		q.d_vpp = fastdiv((uint32_t)(hw / 4));
		q.count = double(n) * double(hw);
		return launch_l2(k2, lp, q, (cudaStream_t)stream, "bn_train_bwd_l2_kernel");
	}
	fused_plan plan;
	const bool fits = fused_mode() == 2 && shape_ok && plan_fused(plan, kernel, n, c, hw, 1, true, 512);
	if (!fits)
	{
		st = nnf_bn_train_bwd_stats(stream, bsums, nullptr, dy, x, gamma, beta, saved, acts, n_acts, n, c, hw, workspace, workspace_bytes);
		if (st != NNF_OK)
			return st;
		return nnf_bn_train_bwd_apply(stream, dx, dy, x, gamma, beta, saved, bsums, bsums, double(n) * double(hw), acts, n_acts,
			grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope, mean, invsigma, entry_count, n, c, hw, add_to_destination);
	}
	fused_params p = {};
	p.x = x; p.dy = dy; p.out = dx; p.gamma = gamma; p.beta = beta; p.saved = const_cast<float *>(saved); p.sums = bsums;
	p.grad_gamma = grad_gamma; p.grad_beta = grad_beta; p.grad_mean = grad_mean; p.grad_invsigma = grad_invsigma; p.grad_slope = grad_slope;
	p.mean = mean; p.invsigma = invsigma; p.entry_count = entry_count;
	p.add = add_to_destination ? 1 : 0;
	p.chain = chain;
	p.n = (uint32_t)n; p.c = (uint32_t)c; p.hw = (uint32_t)hw;
	p.planes_per_cta = plan.planes_per_cta;
	p.cluster = (uint32_t)plan.cluster;
	p.nbuf = 1;
	p.slab_floats = (uint32_t)(plan.planes_per_cta * hw);
	p.d_vpp = fastdiv((uint32_t)(hw / 4));
	p.count = double(n) * double(hw);
	p.error = error_word();
	p.stagger_ns = getenv("NNF_FUSED_STAGGER_NS") ? (uint32_t)atoi(getenv("NNF_FUSED_STAGGER_NS")) : 0;
	{
		const char * t = getenv("NNF_FUSED_TRACE"); // tuning aid: address of a device buffer, as a decimal number
		p.trace = t ? reinterpret_cast<unsigned long long *>(strtoull(t, nullptr, 10)) : nullptr;
	}
	return launch_fused(kernel, plan, p, (cudaStream_t)stream, "bn_train_bwd_cluster_kernel");
}
