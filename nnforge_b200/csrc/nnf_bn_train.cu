// Training-mode batch norm fused with the activation chain that follows it.
//
// Forward : stats kernel (read x once) -> [2C-float all-reduce between GPUs] -> apply kernel (the
//           streaming kernel of nnf_elementwise.cu with mean/invstd derived from the sums in its
//           prologue; read x, write y).
// Backward: bwd-stats kernel (read x, dy; recompute the chain; per-channel sums) -> [2C-float
//           all-reduce] -> bwd-apply kernel (read x, dy; write dx).
// HBM-bound. Algorithmic bytes per element: forward 8 (x in, y out), backward 12 (x, dy in, dx out);
// this two-kernel form moves 12 and 20 because x (and dy) are read twice.
//
// Per-channel reductions: each CTA owns (channel, slice of entries); threads accumulate fp32
// partials over ~100 elements each, the cross-thread and cross-CTA combination is done in double in
// a fixed order (warp shuffles, shared memory, then a second tiny kernel over the per-CTA partials in
// the workspace), so results are deterministic and independent of the grid.
#include "nnf_common.cuh"

#include <mutex>
#include <stdlib.h>

namespace nnf
{
	namespace
	{
		constexpr int kThreads = 256;
		constexpr int kMaxSplit = 64;   // CTAs per channel (upper bound, sizes the workspace)
		constexpr int kSums = 3;        // partial sums per channel and CTA
		constexpr int kLoads = 4;       // independent 128-bit loads in flight per thread (statistics kernels)
		constexpr int kLoads2 = 2;      // same for the kernels that stream two tensors

		__device__ __forceinline__ double warp_sum_d(double v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			return v;
		}

		// Block-wide sum of up to kSums doubles; result valid in thread 0.
		template <int K>
		__device__ __forceinline__ void block_sum_d(double (&v)[K], double * s_red)
		{
			const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
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
			if (threadIdx.x == 0)
			{
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					double t = 0.0;
					for (int i = 0; i < kThreads / 32; ++i)
						t += s_red[i * K + k];
					v[k] = t;
				}
			}
		}

		struct chan_geom
		{
			uint32_t n, c, hw;
			uint32_t split;          // CTAs per channel
			uint32_t entries_per_cta;
			fastdiv d_vpp;           // vectors (or elements) per plane
			int vec;                 // 128-bit loads possible (hw % 4 == 0 and aligned base)
		};

		// workspace layout: double partial[c][split][kSums]
		__global__ void __launch_bounds__(kThreads) bn_stats_kernel(double * partial, const float * x, chan_geom g)
		{
			__shared__ double s_red[(kThreads / 32) * 2];
			const uint32_t ch = blockIdx.x / g.split;
			const uint32_t sp = blockIdx.x - ch * g.split;
			const uint32_t e0 = sp * g.entries_per_cta;
			const uint32_t e1 = min(e0 + g.entries_per_cta, g.n);
			float s = 0.0F, q = 0.0F;
			if (e0 < e1)
			{
				const uint32_t per_plane = g.vec ? (g.hw >> 2) : g.hw;
				const uint32_t total = (e1 - e0) * per_plane;
				const size_t entry_stride = size_t(g.c) * g.hw;
				const float * base = x + (size_t(e0) * g.c + ch) * g.hw;
				// kLoads independent loads are issued before any is consumed: with one load in flight per
				// thread an SM holds too few bytes in flight to cover the HBM latency
				for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kThreads * kLoads)
				{
					if (g.vec)
					{
						float4 a[kLoads];
						#pragma unroll
						for (int u = 0; u < kLoads; ++u)
						{
							const uint32_t i = i0 + u * kThreads;
							a[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
							if (i < total)
							{
								const uint32_t lp = g.d_vpp.div(i);
								a[u] = __ldg(reinterpret_cast<const float4 *>(base + lp * entry_stride) + (i - lp * per_plane)); // default policy: stays in L2
							}
						}
						#pragma unroll
						for (int u = 0; u < kLoads; ++u)
						{
							s += (a[u].x + a[u].y) + (a[u].z + a[u].w);
							q += (a[u].x * a[u].x + a[u].y * a[u].y) + (a[u].z * a[u].z + a[u].w * a[u].w);
						}
					}
					else
					{
						float a[kLoads];
						#pragma unroll
						for (int u = 0; u < kLoads; ++u)
						{
							const uint32_t i = i0 + u * kThreads;
							a[u] = 0.0F;
							if (i < total)
							{
								const uint32_t lp = g.d_vpp.div(i);
								a[u] = __ldg(base + lp * entry_stride + (i - lp * per_plane));
							}
						}
						#pragma unroll
						for (int u = 0; u < kLoads; ++u)
						{
							s += a[u];
							q += a[u] * a[u];
						}
					}
				}
			}
			double acc[2] = {double(s), double(q)};
			block_sum_d<2>(acc, s_red);
			if (threadIdx.x == 0)
			{
				double * out = partial + (size_t(ch) * g.split + sp) * kSums;
				out[0] = acc[0];
				out[1] = acc[1];
			}
		}

		// sums[k*c + ch] (+)= float(sum over splits of partial[ch][split][k]), k < count
		// copy (may be null) receives the first copy_count sums too: the buffer a caller all-reduces
		__global__ void bn_reduce_partials_kernel(float * sums, const double * partial, uint32_t c, uint32_t split, int count, int accumulate,
			float * copy = nullptr, int copy_count = 0)
		{
			const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
			if (ch >= c)
				return;
			for (int k = 0; k < count; ++k)
			{
				double t = 0.0;
				for (uint32_t sp = 0; sp < split; ++sp)
					t += partial[(size_t(ch) * split + sp) * kSums + k];
				float * out = sums + size_t(k) * c + ch;
				*out = accumulate ? *out + float(t) : float(t);
				if (copy && k < copy_count)
					copy[size_t(k) * c + ch] = float(t);
			}
		}

		// The same reduction fused with the publication of its first `publish_count` sums to every rank's
		// peer buffer (see nnf_peer.cu): one CTA, so that a single barrier tells when all stores are issued.
		__global__ void __launch_bounds__(1024) bn_reduce_publish_kernel(float * sums, const double * partial, uint32_t c, uint32_t split, int count,
			float * copy, int copy_count, peer_dst dst, int publish_count)
		{
			for (uint32_t ch = threadIdx.x; ch < c; ch += blockDim.x)
				for (int k = 0; k < count; ++k)
				{
					double t = 0.0;
					for (uint32_t sp = 0; sp < split; ++sp)
						t += partial[(size_t(ch) * split + sp) * kSums + k];
					const float v = float(t);
					sums[size_t(k) * c + ch] = v;
					if (copy && k < copy_count)
						copy[size_t(k) * c + ch] = v;
					if (k < publish_count)
						peer_store(dst, k * c + ch, v);
				}
			peer_raise_flags(dst);
		}

		// PReLU slope gradient partials: sum dy * (x >= 0 ? 0 : x) per (channel, slice of entries)
		__global__ void __launch_bounds__(kThreads) prelu_dslope_kernel(double * partial, const float * dy, const float * x, chan_geom g)
		{
			__shared__ double s_red[kThreads / 32];
			const uint32_t ch = blockIdx.x / g.split;
			const uint32_t sp = blockIdx.x - ch * g.split;
			const uint32_t e0 = sp * g.entries_per_cta;
			const uint32_t e1 = min(e0 + g.entries_per_cta, g.n);
			float s = 0.0F;
			if (e0 < e1)
			{
				const uint32_t per_plane = g.vec ? (g.hw >> 2) : g.hw;
				const uint32_t total = (e1 - e0) * per_plane;
				const size_t entry_stride = size_t(g.c) * g.hw;
				const size_t off0 = (size_t(e0) * g.c + ch) * g.hw;
				for (uint32_t i = threadIdx.x; i < total; i += kThreads)
				{
					const uint32_t lp = g.d_vpp.div(i);
					const uint32_t v = i - lp * per_plane;
					const size_t off = off0 + lp * entry_stride;
					if (g.vec)
					{
						const float4 a = ld_stream(reinterpret_cast<const float4 *>(x + off) + v);
						const float4 d = ld_stream(reinterpret_cast<const float4 *>(dy + off) + v);
						s += d.x * (a.x >= 0.0F ? 0.0F : a.x);
						s += d.y * (a.y >= 0.0F ? 0.0F : a.y);
						s += d.z * (a.z >= 0.0F ? 0.0F : a.z);
						s += d.w * (a.w >= 0.0F ? 0.0F : a.w);
					}
					else
					{
						const float a = x[off + v];
						s += dy[off + v] * (a >= 0.0F ? 0.0F : a);
					}
				}
			}
			double acc[1] = {double(s)};
			block_sum_d<1>(acc, s_red);
			if (threadIdx.x == 0)
				partial[(size_t(ch) * g.split + sp) * kSums] = acc[0];
		}

		struct bwd_params
		{
			const float * dy;
			const float * x;
			const float * gamma;
			const float * beta;
			const float * saved;   // {mean, invstd}
			act_chain chain;
			// bwd-apply only
			float * dx;
			const float * gsums;   // global {sum du, sum du*xhat}
			const float * bsums;   // local  {sum du, sum du*xhat, sum dslope}
			double count_total;
			float * grad_gamma, * grad_beta, * grad_mean, * grad_invsigma, * grad_slope;
			const float * mean, * invsigma;
			float entry_count;
			int add;
			peer_src peer;         // peer.mine != null: gsums come from the peer buffer
		};

		template <int A0, int A1>
		__global__ void __launch_bounds__(kThreads) bn_bwd_stats_kernel(double * partial, const bwd_params p, chan_geom g)
		{
			__shared__ double s_red[(kThreads / 32) * 3];
			// channels in descending order: whatever ran before (the forward kernels walk the channels upwards)
			// left the highest channels of x in L2; bn_bwd_apply_kernel then walks upwards again
			const uint32_t ch = g.c - 1 - blockIdx.x / g.split;
			const uint32_t sp = blockIdx.x % g.split;
			const uint32_t e0 = sp * g.entries_per_cta;
			const uint32_t e1 = min(e0 + g.entries_per_cta, g.n);
			const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + g.c + ch);
			const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
			const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			const float slope = chain_slope(p.chain, ch);
			float sb = 0.0F, sg = 0.0F, ss = 0.0F;
			auto element = [&](float x, float dy)
			{
				const float u = __fadd_rn(__fmul_rn(x, mult), add);
				float term;
				const float du = chain_backward<A0, A1>(p.chain, u, dy, slope, term);
				const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
				sb += du;
				sg += du * xhat;
				ss += term;
			};
			if (e0 < e1)
			{
				const uint32_t per_plane = g.vec ? (g.hw >> 2) : g.hw;
				const uint32_t total = (e1 - e0) * per_plane;
				const size_t entry_stride = size_t(g.c) * g.hw;
				const size_t off0 = (size_t(e0) * g.c + ch) * g.hw;
				for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kThreads * kLoads2)
				{
					if (g.vec)
					{
						float4 a[kLoads2], d[kLoads2];
						#pragma unroll
						for (int u = 0; u < kLoads2; ++u)
						{
							const uint32_t i = i0 + u * kThreads;
							if (i < total)
							{
								const uint32_t lp = g.d_vpp.div(i);
								const size_t off = off0 + lp * entry_stride;
								a[u] = __ldg(reinterpret_cast<const float4 *>(p.x + off) + (i - lp * per_plane));   // default policy: the channels
								d[u] = __ldg(reinterpret_cast<const float4 *>(p.dy + off) + (i - lp * per_plane));  // read last stay in L2 for bn_bwd_apply_kernel
							}
						}
						#pragma unroll
						for (int u = 0; u < kLoads2; ++u)
							if (i0 + u * kThreads < total)
							{
								element(a[u].x, d[u].x); element(a[u].y, d[u].y); element(a[u].z, d[u].z); element(a[u].w, d[u].w);
							}
					}
					else
					{
						#pragma unroll
						for (int u = 0; u < kLoads2; ++u)
						{
							const uint32_t i = i0 + u * kThreads;
							if (i < total)
							{
								const uint32_t lp = g.d_vpp.div(i);
								const size_t off = off0 + lp * entry_stride + (i - lp * per_plane);
								element(__ldg(p.x + off), __ldg(p.dy + off));
							}
						}
					}
				}
			}
			double acc[3] = {double(sb), double(sg), double(ss)};
			block_sum_d<3>(acc, s_red);
			if (threadIdx.x == 0)
			{
				double * out = partial + (size_t(ch) * g.split + sp) * kSums;
				out[0] = acc[0];
				out[1] = acc[1];
				out[2] = acc[2];
			}
		}

		// dx (+)= mult * (du - dbeta/m - xhat*dgamma/m); one CTA per (channel, slice of entries).
		template <int A0, int A1>
		__global__ void __launch_bounds__(kThreads) bn_bwd_apply_kernel(const bwd_params p, chan_geom g)
		{
			// channels in ascending order: bn_bwd_stats_kernel, which ran just before, walked them downwards with
			// default-policy loads, so the channels it read last (the lowest, ~100 MB still in L2) come first
			const uint32_t ch = blockIdx.x / g.split;
			const uint32_t sp = blockIdx.x % g.split;
			const uint32_t e0 = sp * g.entries_per_cta;
			const uint32_t e1 = min(e0 + g.entries_per_cta, g.n);
			const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + g.c + ch);
			const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
			const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			const float slope = chain_slope(p.chain, ch);
			float gb, gg;
			if (p.peer.mine)
			{
				peer_wait(p.peer);
				gb = peer_sum(p.peer, ch);
				gg = peer_sum(p.peer, g.c + ch);
			}
			else
			{
				gb = __ldg(p.gsums + ch);
				gg = __ldg(p.gsums + g.c + ch);
			}
			const float c2 = float(double(gb) / p.count_total);
			const float c3 = float(double(gg) / p.count_total);

			if (sp == 0 && threadIdx.x == 0)
			{
				// per-channel gradients accumulate the LOCAL sums (batch_norm_layer_updater_cuda.cu:138-139, 167-182)
				if (p.grad_beta) p.grad_beta[ch] += p.bsums[ch];
				if (p.grad_gamma) p.grad_gamma[ch] += p.bsums[g.c + ch];
				if (p.grad_slope) p.grad_slope[ch] += p.bsums[2 * g.c + ch];
				if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (mean - p.mean[ch]);
				if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (invstd - p.invsigma[ch]);
			}

			auto element = [&](float x, float dy, float old) -> float
			{
				const float u = __fadd_rn(__fmul_rn(x, mult), add);
				float term;
				const float du = chain_backward<A0, A1>(p.chain, u, dy, slope, term);
				const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
				const float r = mult * ((du - c2) - xhat * c3);
				return p.add ? old + r : r;
			};
			if (e0 >= e1)
				return;
			const uint32_t per_plane = g.vec ? (g.hw >> 2) : g.hw;
			const uint32_t total = (e1 - e0) * per_plane;
			const size_t entry_stride = size_t(g.c) * g.hw;
			const size_t off0 = (size_t(e0) * g.c + ch) * g.hw;
			for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kThreads * kLoads2)
			{
				if (g.vec)
				{
					float4 a[kLoads2], d[kLoads2], o[kLoads2];
					size_t pos[kLoads2];
					#pragma unroll
					for (int u = 0; u < kLoads2; ++u)
					{
						const uint32_t i = i0 + u * kThreads;
						o[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						if (i < total)
						{
							const uint32_t lp = g.d_vpp.div(i);
							pos[u] = off0 + lp * entry_stride + size_t(i - lp * per_plane) * 4;
							a[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + pos[u]));
							d[u] = ld_stream(reinterpret_cast<const float4 *>(p.dy + pos[u]));
							if (p.add)
								o[u] = ld_stream(reinterpret_cast<const float4 *>(p.dx + pos[u]));
						}
					}
					#pragma unroll
					for (int u = 0; u < kLoads2; ++u)
						if (i0 + u * kThreads < total)
						{
							const float4 r = make_float4(element(a[u].x, d[u].x, o[u].x), element(a[u].y, d[u].y, o[u].y),
								element(a[u].z, d[u].z, o[u].z), element(a[u].w, d[u].w, o[u].w));
							st_stream(reinterpret_cast<float4 *>(p.dx + pos[u]), r);
						}
				}
				else
				{
					#pragma unroll
					for (int u = 0; u < kLoads2; ++u)
					{
						const uint32_t i = i0 + u * kThreads;
						if (i < total)
						{
							const uint32_t lp = g.d_vpp.div(i);
							const size_t off = off0 + lp * entry_stride + (i - lp * per_plane);
							const float old = p.add ? p.dx[off] : 0.0F;
							p.dx[off] = element(p.x[off], p.dy[off], old);
						}
					}
				}
			}
		}

		// Training-mode normalisation + activation chain, one CTA per (channel, slice of entries), channels in
		// DESCENDING order. It runs right after bn_stats_kernel, which walked the channels in ascending order
		// with default-policy loads: the ~100 MB that kernel read last are still in L2 and are consumed first
		// here, so part of the second read of x never reaches HBM. (The flat streaming kernel of
		// nnf_elementwise.cu computes the same values in memory order and is used for shapes this one does
		// not take.)
		struct apply_params
		{
			float * y;
			const float * x;
			const float * gamma;
			const float * beta;
			const float * sums;
			float * saved;
			double count_total;
			float eps;
			act_chain chain;
			peer_src peer;         // peer.mine != null: the sums of all ranks are taken from the peer buffer
		};

		template <int A0, int A1>
		__global__ void __launch_bounds__(kThreads) bn_apply_channel_kernel(const apply_params p, chan_geom g)
		{
			const uint32_t ch = g.c - 1 - blockIdx.x / g.split;
			const uint32_t sp = blockIdx.x % g.split;
			const uint32_t e0 = sp * g.entries_per_cta;
			const uint32_t e1 = min(e0 + g.entries_per_cta, g.n);
			// batch statistics of this channel: biased variance from the (all-reduced) sum and sum of squares
			float fs, fq;
			if (p.peer.mine)
			{
				peer_wait(p.peer);
				fs = peer_sum(p.peer, ch);
				fq = peer_sum(p.peer, g.c + ch);
			}
			else
			{
				fs = __ldg(p.sums + ch);
				fq = __ldg(p.sums + g.c + ch);
			}
			const double m = double(fs) / p.count_total;
			double var = double(fq) / p.count_total - m * m;
			var = var < 0.0 ? 0.0 : var;
			const float mean = float(m);
			const float invstd = float(1.0 / sqrt(var + double(p.eps)));
			if (sp == 0 && threadIdx.x == 0 && p.saved)
			{
				p.saved[ch] = mean;
				p.saved[g.c + ch] = invstd;
			}
			const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
			const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			const float slope = chain_slope(p.chain, ch);
			if (e0 >= e1)
				return;
			const uint32_t per_plane = g.hw >> 2;
			const uint32_t total = (e1 - e0) * per_plane;
			const size_t entry_stride = size_t(g.c) * g.hw;
			const size_t off0 = (size_t(e0) * g.c + ch) * g.hw;
			for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kThreads * kLoads)
			{
				float4 a[kLoads];
				size_t pos[kLoads];
				#pragma unroll
				for (int u = 0; u < kLoads; ++u)
				{
					const uint32_t i = i0 + u * kThreads;
					if (i < total)
					{
						const uint32_t lp = g.d_vpp.div(i);
						pos[u] = off0 + lp * entry_stride + size_t(i - lp * per_plane) * 4;
						a[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + pos[u]));
					}
				}
				#pragma unroll
				for (int u = 0; u < kLoads; ++u)
					if (i0 + u * kThreads < total)
					{
						float4 o;
						o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].x, mult), add), slope);
						o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].y, mult), add), slope);
						o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].z, mult), add), slope);
						o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].w, mult), add), slope);
						st_stream(reinterpret_cast<float4 *>(p.y + pos[u]), o);
					}
			}
		}

		// CTAs of `kernel` that one SM holds at once (queried once per kernel and cached).
		template <class Kernel>
		int resident_ctas_per_sm(Kernel kernel)
		{
			static int cached = 0;
			if (cached == 0)
			{
				int v = 0;
				if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, kernel, kThreads, 0) != cudaSuccess || v < 1)
				{
					cudaGetLastError();
					v = 4;
				}
				cached = v;
			}
			return cached;
		}

		int make_chan_geom(chan_geom& g, const char * who, int64_t n, int64_t c, int64_t hw, bool vec_ok, int ctas_per_sm, int waves)
		{
			if (n > 0x7fffffff || c > 0x7fffffff || hw > 0x7fffffff || n * hw > kMaxElemsPerLaunch)
				return set_error(NNF_ERR_UNSUPPORTED, "%s: n*hw must stay below 2^31 per channel", who);
			g.n = (uint32_t)n; g.c = (uint32_t)c; g.hw = (uint32_t)hw;
			g.vec = (vec_ok && (hw % 4 == 0)) ? 1 : 0;
			// One wave: as many CTAs as the machine holds at once and no more. A grid slightly larger than
			// that would run a second, nearly empty wave and double the kernel's duration; with more
			// channels than resident CTAs there are many waves of equal CTAs and the tail is small.
			// `waves` resident waves of CTAs. Measured on B200 (x[256,256,28,28]): the reducing kernels are
			// best with 1-2 waves (each CTA ends with a block reduction and a partial-sum store), the
			// streaming backward-apply kernel with 8 (95% of the measured copy bandwidth against 88% with
			// one wave: CTAs that start at different times mix their loads and stores instead of moving in
			// lockstep through load / compute / store phases).
			if (tune().channel_waves > 0)
				waves = tune().channel_waves;
			int64_t split = (int64_t(sm_count()) * ctas_per_sm * (waves < 1 ? 1 : waves)) / c;
			const int64_t max_by_work = (n * hw) / 8192 > 0 ? (n * hw) / 8192 : 1;
			if (split > max_by_work) split = max_by_work;
			if (split > n) split = n;
			if (split > kMaxSplit) split = kMaxSplit;
			if (split < 1) split = 1;
			g.entries_per_cta = (uint32_t)div_up(n, split);
			g.split = (uint32_t)div_up(n, g.entries_per_cta);
			g.d_vpp = fastdiv(g.vec ? g.hw / 4 : g.hw);
			return NNF_OK;
		}

		// ---- planes that are not whole float4s (7x7, 13x13, fully connected: H*W % 4 != 0) -----------------------
		// A single plane is then neither 16-byte aligned nor a whole number of vectors, and the kernels above fall
		// back to scalar loads of 49-float runs. `unit` = 4 / gcd(H*W, 4) adjacent channels of one entry do form an
		// aligned run of whole vectors, so here a CTA owns a GROUP of G channels (a multiple of `unit`) and a slice of
		// entries; the group's run of G*H*W floats per entry is read with coalesced 128-bit loads. A thread owns the
		// same vector positions of the run in every entry, so the channel of each of its elements - and every
		// per-channel constant - is fixed for the whole loop and sits in registers, and it accumulates per POSITION;
		// at the end the positions are folded per channel through shared memory in a fixed order.
		constexpr int kGroupMaxRun = 2048;      // floats of one group's run (R <= 2 vectors per thread)

		struct group_geom
		{
			uint32_t n, c, hw;
			uint32_t group;            // channels per group
			uint32_t groups;
			uint32_t split, entries_per_cta;
			int vectors_per_thread;    // 1 or 2
			fastdiv d_hw;
		};

		// false: the shape keeps the per-channel kernels
		bool make_group_geom(group_geom& g, int64_t n, int64_t c, int64_t hw, bool aligned)
		{
			if (!aligned || hw % 4 == 0 || tune().no_grouped == 1)
				return false;
			const int64_t unit = (hw % 2 == 0) ? 2 : 4;
			const int64_t vpu = unit * hw / 4;        // vectors of one unit of channels
			if (c % unit != 0 || vpu > 2 * kThreads || n > 0x7fffffff || c > 0x7fffffff)
				return false;
			const int64_t k1 = kThreads / vpu, k2 = (2 * kThreads) / vpu;
			int r = 1;
			int64_t k = k1;
			if (k1 == 0 || double(k2 * vpu) / (2 * kThreads) > double(k1 * vpu) / kThreads + 0.1)
			{
				r = 2;
				k = k2;
			}
			int64_t group = unit * k;
			if (group > c)
				group = c;
			if (group > 1024)   // kGroupMaxChannels: the per-group tables of bn_apply_grouped_kernel
				group = 1024;
			g.n = (uint32_t)n; g.c = (uint32_t)c; g.hw = (uint32_t)hw;
			g.group = (uint32_t)group;
			g.groups = (uint32_t)div_up(c, group);
			g.vectors_per_thread = r;
			const int64_t waves = tune().group_waves > 0 ? tune().group_waves : 1;
			int64_t split = div_up(int64_t(sm_count()) * 8 * waves, g.groups);
			if (split > n / 4) split = n / 4;
			if (split > kMaxSplit) split = kMaxSplit;
			if (split < 1) split = 1;
			g.entries_per_cta = (uint32_t)div_up(n, split);
			g.split = (uint32_t)div_up(n, g.entries_per_cta);
			g.d_hw = fastdiv((uint32_t)hw);
			return true;
		}

		struct group_cta
		{
			uint32_t ch0, channels, vectors, sp, e0, e1;
			size_t stride4;            // float4s between the same position of consecutive entries
			size_t base4;              // float4 offset of the group's run in entry e0
		};

		// descending: the groups are walked downwards (a kernel that follows one that walked upwards finds the data
		// that kernel touched last, up to the size of L2, still cached)
		__device__ __forceinline__ group_cta group_locate(const group_geom& g, bool descending = false)
		{
			group_cta t;
			const uint32_t walk = blockIdx.x / g.split;
			const uint32_t grp = descending ? g.groups - 1 - walk : walk;
			t.sp = blockIdx.x - walk * g.split;
			t.ch0 = grp * g.group;
			t.channels = min(g.group, g.c - t.ch0);
			t.vectors = (t.channels * g.hw) >> 2;
			t.e0 = t.sp * g.entries_per_cta;
			t.e1 = min(t.e0 + g.entries_per_cta, g.n);
			t.stride4 = (size_t(g.c) * g.hw) >> 2;
			t.base4 = ((size_t(t.e0) * g.c + t.ch0) * g.hw) >> 2;
			return t;
		}

		// per-channel sum of K position arrays held in shared memory -> this CTA's partials. Eight lanes share a
		// channel: each sums every eighth position in double, a three-step butterfly joins them (a fixed order).
		template <int K>
		__device__ __forceinline__ void group_fold(double * partial, const float (*s_pos)[kGroupMaxRun], const group_geom& g, const group_cta& t)
		{
			constexpr uint32_t kLanes = 8;
			const uint32_t lane = threadIdx.x % kLanes;
			for (uint32_t first = 0; first < t.channels; first += kThreads / kLanes)
			{
				const uint32_t ch = first + threadIdx.x / kLanes;
				double acc[K];
				#pragma unroll
				for (int k = 0; k < K; ++k)
					acc[k] = 0.0;
				if (ch < t.channels)
					for (uint32_t i = lane; i < g.hw; i += kLanes)
					{
						#pragma unroll
						for (int k = 0; k < K; ++k)
							acc[k] += double(s_pos[k][ch * g.hw + i]);
					}
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 4);
					acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 2);
					acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 1);
				}
				if (ch < t.channels && lane == 0)
				{
					double * out = partial + (size_t(t.ch0 + ch) * g.split + t.sp) * kSums;
					#pragma unroll
					for (int k = 0; k < K; ++k)
						out[k] = acc[k];
				}
			}
		}

		template <int R>
		__global__ void __launch_bounds__(kThreads) bn_stats_grouped_kernel(double * partial, const float * x, const group_geom g)
		{
			__shared__ float s_pos[2][kGroupMaxRun];
			constexpr int U = 4;   // entries in flight
			const group_cta t = group_locate(g);
			float s[R][4], q[R][4];
			#pragma unroll
			for (int r = 0; r < R; ++r)
				#pragma unroll
				for (int j = 0; j < 4; ++j)
					s[r][j] = q[r][j] = 0.0F;
			const float4 * base = reinterpret_cast<const float4 *>(x) + t.base4;
			for (uint32_t e = t.e0; e < t.e1; e += U)
			{
				float4 a[U][R];
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						a[u][r] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						if (e + u < t.e1 && v < t.vectors)
							a[u][r] = __ldg(base + size_t(e + u - t.e0) * t.stride4 + v);
					}
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						s[r][0] += a[u][r].x; s[r][1] += a[u][r].y; s[r][2] += a[u][r].z; s[r][3] += a[u][r].w;
						q[r][0] = fmaf(a[u][r].x, a[u][r].x, q[r][0]); q[r][1] = fmaf(a[u][r].y, a[u][r].y, q[r][1]);
						q[r][2] = fmaf(a[u][r].z, a[u][r].z, q[r][2]); q[r][3] = fmaf(a[u][r].w, a[u][r].w, q[r][3]);
					}
			}
			#pragma unroll
			for (int r = 0; r < R; ++r)
			{
				const uint32_t v = threadIdx.x + r * kThreads;
				if (v < t.vectors)
					#pragma unroll
					for (int j = 0; j < 4; ++j)
					{
						s_pos[0][v * 4 + j] = s[r][j];
						s_pos[1][v * 4 + j] = q[r][j];
					}
			}
			__syncthreads();
			group_fold<2>(partial, s_pos, g, t);
		}

		// PReLU slope gradient partials on channel groups: sum dy * (x >= 0 ? 0 : x) per position, folded per channel
		template <int R>
		__global__ void __launch_bounds__(kThreads) prelu_dslope_grouped_kernel(double * partial, const float * dy, const float * x, const group_geom g)
		{
			__shared__ float s_pos[1][kGroupMaxRun];
			constexpr int U = 2;
			const group_cta t = group_locate(g);
			float acc[R][4];
			#pragma unroll
			for (int r = 0; r < R; ++r)
				#pragma unroll
				for (int j = 0; j < 4; ++j)
					acc[r][j] = 0.0F;
			const float4 * bx = reinterpret_cast<const float4 *>(x) + t.base4;
			const float4 * bd = reinterpret_cast<const float4 *>(dy) + t.base4;
			for (uint32_t e = t.e0; e < t.e1; e += U)
			{
				float4 a[U][R], d[U][R];
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						a[u][r] = d[u][r] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						if (e + u < t.e1 && v < t.vectors)
						{
							const size_t off = size_t(e + u - t.e0) * t.stride4 + v;
							a[u][r] = ld_stream(bx + off);
							d[u][r] = ld_stream(bd + off);
						}
					}
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						// parametric_rectified_linear_layer_updater_plain.cpp:177-180
						acc[r][0] += d[u][r].x * (a[u][r].x >= 0.0F ? 0.0F : a[u][r].x);
						acc[r][1] += d[u][r].y * (a[u][r].y >= 0.0F ? 0.0F : a[u][r].y);
						acc[r][2] += d[u][r].z * (a[u][r].z >= 0.0F ? 0.0F : a[u][r].z);
						acc[r][3] += d[u][r].w * (a[u][r].w >= 0.0F ? 0.0F : a[u][r].w);
					}
			}
			#pragma unroll
			for (int r = 0; r < R; ++r)
			{
				const uint32_t v = threadIdx.x + r * kThreads;
				if (v < t.vectors)
					#pragma unroll
					for (int j = 0; j < 4; ++j)
						s_pos[0][v * 4 + j] = acc[r][j];
			}
			__syncthreads();
			group_fold<1>(partial, s_pos, g, t);
		}

		// the constants of one owned element
		struct group_elem
		{
			float mean, invstd, mult, add, slope, c2, c3;
		};

		template <int R>
		__device__ __forceinline__ void group_constants(group_elem (&k)[R][4], const bwd_params& p, const group_geom& g, const group_cta& t, bool with_sums)
		{
			#pragma unroll
			for (int r = 0; r < R; ++r)
			{
				const uint32_t v = threadIdx.x + r * kThreads;
				#pragma unroll
				for (int j = 0; j < 4; ++j)
				{
					const uint32_t pos = min(v * 4 + j, t.channels * g.hw - 1);
					const uint32_t ch = t.ch0 + g.d_hw.div(pos);
					group_elem& el = k[r][j];
					el.mean = __ldg(p.saved + ch);
					el.invstd = __ldg(p.saved + g.c + ch);
					el.mult = __fmul_rn(__ldg(p.gamma + ch), el.invstd);
					el.add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(el.mult, el.mean));
					el.slope = chain_slope(p.chain, ch);
					el.c2 = el.c3 = 0.0F;
					if (with_sums)
					{
						el.c2 = float(double(__ldg(p.gsums + ch)) / p.count_total);
						el.c3 = float(double(__ldg(p.gsums + g.c + ch)) / p.count_total);
					}
				}
			}
		}

		template <int A0, int A1, int R>
		__global__ void __launch_bounds__(kThreads) bn_bwd_stats_grouped_kernel(double * partial, const bwd_params p, const group_geom g)
		{
			__shared__ float s_pos[3][kGroupMaxRun];
			constexpr int U = 2;
			const group_cta t = group_locate(g, true);
			group_elem k[R][4];
			group_constants<R>(k, p, g, t, false);
			float sb[R][4], sg[R][4], ss[R][4];
			#pragma unroll
			for (int r = 0; r < R; ++r)
				#pragma unroll
				for (int j = 0; j < 4; ++j)
					sb[r][j] = sg[r][j] = ss[r][j] = 0.0F;
			const float4 * bx = reinterpret_cast<const float4 *>(p.x) + t.base4;
			const float4 * bd = reinterpret_cast<const float4 *>(p.dy) + t.base4;
			for (uint32_t e = t.e0; e < t.e1; e += U)
			{
				float4 a[U][R], d[U][R];
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						a[u][r] = d[u][r] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						if (e + u < t.e1 && v < t.vectors)
						{
							const size_t off = size_t(e + u - t.e0) * t.stride4 + v;
							a[u][r] = __ldg(bx + off);
							d[u][r] = __ldg(bd + off);
						}
					}
				#pragma unroll
				for (int u = 0; u < U; ++u)
					if (e + u < t.e1)
					{
						#pragma unroll
						for (int r = 0; r < R; ++r)
						{
							const float xs[4] = {a[u][r].x, a[u][r].y, a[u][r].z, a[u][r].w};
							const float ds[4] = {d[u][r].x, d[u][r].y, d[u][r].z, d[u][r].w};
							#pragma unroll
							for (int j = 0; j < 4; ++j)
							{
								const group_elem& el = k[r][j];
								const float uu = __fadd_rn(__fmul_rn(xs[j], el.mult), el.add);
								float term;
								const float du = chain_backward<A0, A1>(p.chain, uu, ds[j], el.slope, term);
								const float xhat = __fmul_rn(__fsub_rn(xs[j], el.mean), el.invstd);
								sb[r][j] += du;
								sg[r][j] += du * xhat;
								ss[r][j] += term;
							}
						}
					}
			}
			#pragma unroll
			for (int r = 0; r < R; ++r)
			{
				const uint32_t v = threadIdx.x + r * kThreads;
				if (v < t.vectors)
					#pragma unroll
					for (int j = 0; j < 4; ++j)
					{
						s_pos[0][v * 4 + j] = sb[r][j];
						s_pos[1][v * 4 + j] = sg[r][j];
						s_pos[2][v * 4 + j] = ss[r][j];
					}
			}
			__syncthreads();
			group_fold<3>(partial, s_pos, g, t);
		}

		template <int A0, int A1, int R>
		__global__ void __launch_bounds__(kThreads) bn_bwd_apply_grouped_kernel(const bwd_params p, const group_geom g)
		{
			constexpr int U = 2;
			const group_cta t = group_locate(g);
			if (t.sp == 0)
				for (uint32_t i = threadIdx.x; i < t.channels; i += kThreads)
				{
					// per-channel gradients accumulate the LOCAL sums (batch_norm_layer_updater_cuda.cu:138-139, 167-182)
					const uint32_t ch = t.ch0 + i;
					if (p.grad_beta) p.grad_beta[ch] += p.bsums[ch];
					if (p.grad_gamma) p.grad_gamma[ch] += p.bsums[g.c + ch];
					if (p.grad_slope) p.grad_slope[ch] += p.bsums[2 * g.c + ch];
					if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (__ldg(p.saved + ch) - p.mean[ch]);
					if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (__ldg(p.saved + g.c + ch) - p.invsigma[ch]);
				}
			group_elem k[R][4];
			group_constants<R>(k, p, g, t, true);
			const float4 * bx = reinterpret_cast<const float4 *>(p.x) + t.base4;
			const float4 * bd = reinterpret_cast<const float4 *>(p.dy) + t.base4;
			float4 * bo = reinterpret_cast<float4 *>(p.dx) + t.base4;
			for (uint32_t e = t.e0; e < t.e1; e += U)
			{
				float4 a[U][R], d[U][R], o[U][R];
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						o[u][r] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						if (e + u < t.e1 && v < t.vectors)
						{
							const size_t off = size_t(e + u - t.e0) * t.stride4 + v;
							a[u][r] = ld_stream(bx + off);
							d[u][r] = ld_stream(bd + off);
							if (p.add)
								o[u][r] = ld_stream(bo + off);
						}
					}
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						if (e + u < t.e1 && v < t.vectors)
						{
							const float xs[4] = {a[u][r].x, a[u][r].y, a[u][r].z, a[u][r].w};
							const float ds[4] = {d[u][r].x, d[u][r].y, d[u][r].z, d[u][r].w};
							const float os[4] = {o[u][r].x, o[u][r].y, o[u][r].z, o[u][r].w};
							float rs[4];
							#pragma unroll
							for (int j = 0; j < 4; ++j)
							{
								const group_elem& el = k[r][j];
								const float uu = __fadd_rn(__fmul_rn(xs[j], el.mult), el.add);
								float term;
								const float du = chain_backward<A0, A1>(p.chain, uu, ds[j], el.slope, term);
								const float xhat = __fmul_rn(__fsub_rn(xs[j], el.mean), el.invstd);
								const float res = el.mult * ((du - el.c2) - xhat * el.c3);
								rs[j] = p.add ? os[j] + res : res;
							}
							st_stream(bo + size_t(e + u - t.e0) * t.stride4 + v, make_float4(rs[0], rs[1], rs[2], rs[3]));
						}
					}
			}
		}

		constexpr int kGroupMaxChannels = 1024;   // channels of one group (reached by fully connected shapes, H*W = 1)

		// Training-mode normalisation + activation chain on a channel group: scale and shift of the group's channels
		// are derived once per CTA into shared memory (same expressions as bn_apply_channel_kernel), every thread then
		// keeps the constants of the elements it owns in registers.
		template <int A0, int A1, int R>
		__global__ void __launch_bounds__(kThreads) bn_apply_grouped_kernel(const apply_params p, const group_geom g)
		{
			__shared__ float s_mult[kGroupMaxChannels], s_add[kGroupMaxChannels];
			constexpr int U = 4;
			const group_cta t = group_locate(g, true);
			for (uint32_t i = threadIdx.x; i < t.channels; i += kThreads)
			{
				const uint32_t ch = t.ch0 + i;
				const double m = double(__ldg(p.sums + ch)) / p.count_total;
				double var = double(__ldg(p.sums + g.c + ch)) / p.count_total - m * m;
				var = var < 0.0 ? 0.0 : var;
				const float mean = float(m);
				const float invstd = float(1.0 / sqrt(var + double(p.eps)));
				if (t.sp == 0 && p.saved)
				{
					p.saved[ch] = mean;
					p.saved[g.c + ch] = invstd;
				}
				const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
				s_mult[i] = mult;
				s_add[i] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			}
			__syncthreads();
			float mult[R][4], add[R][4], slope[R][4];
			#pragma unroll
			for (int r = 0; r < R; ++r)
			{
				const uint32_t v = threadIdx.x + r * kThreads;
				#pragma unroll
				for (int j = 0; j < 4; ++j)
				{
					const uint32_t local = g.d_hw.div(min(v * 4 + j, t.channels * g.hw - 1));
					mult[r][j] = s_mult[local];
					add[r][j] = s_add[local];
					slope[r][j] = chain_slope(p.chain, t.ch0 + local);
				}
			}
			const float4 * bx = reinterpret_cast<const float4 *>(p.x) + t.base4;
			float4 * by = reinterpret_cast<float4 *>(p.y) + t.base4;
			for (uint32_t e = t.e0; e < t.e1; e += U)
			{
				float4 a[U][R];
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						if (e + u < t.e1 && v < t.vectors)
							a[u][r] = ld_stream(bx + size_t(e + u - t.e0) * t.stride4 + v);
					}
				#pragma unroll
				for (int u = 0; u < U; ++u)
					#pragma unroll
					for (int r = 0; r < R; ++r)
					{
						const uint32_t v = threadIdx.x + r * kThreads;
						if (e + u < t.e1 && v < t.vectors)
						{
							float4 o;
							o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u][r].x, mult[r][0]), add[r][0]), slope[r][0]);
							o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u][r].y, mult[r][1]), add[r][1]), slope[r][1]);
							o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u][r].z, mult[r][2]), add[r][2]), slope[r][2]);
							o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u][r].w, mult[r][3]), add[r][3]), slope[r][3]);
							st_stream(by + size_t(e + u - t.e0) * t.stride4 + v, o);
						}
					}
			}
		}

		int check_train_args(const char * who, int64_t n, int64_t c, int64_t hw)
		{
			if (n <= 0 || c <= 0 || hw <= 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: bad extents n=%lld c=%lld hw=%lld (training batch norm needs at least one entry)", who, (long long)n, (long long)c, (long long)hw);
			return NNF_OK;
		}
	}
}

using namespace nnf;

extern "C" size_t nnf_bn_train_workspace_bytes(int64_t n, int64_t c, int64_t hw)
{
	if (c <= 0 || n <= 0 || hw <= 0)
		return 0;
	const size_t two_kernel = size_t(c) * kMaxSplit * kSums * sizeof(double);
	const size_t single_launch = chain_workspace_bytes(n, c, hw);
	return two_kernel > single_launch ? two_kernel : single_launch;
}

namespace
{
	int stats_impl(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw,
		void * workspace, size_t workspace_bytes, const peer_dst * publish);
}

extern "C" int nnf_bn_train_stats(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes)
{
	return stats_impl(stream, sums, x, n, c, hw, workspace, workspace_bytes, nullptr);
}

extern "C" int nnf_bn_train_stats_publish(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes, void * const * peer_bufs, int rank, int world, int kmax, uint32_t seq)
{
	peer_dst d;
	int st = make_peer_dst(d, peer_bufs, rank, world, (int)(2 * c), kmax, seq, "nnf_bn_train_stats_publish");
	if (st != NNF_OK)
		return st;
	return stats_impl(stream, sums, x, n, c, hw, workspace, workspace_bytes, &d);
}

namespace
{
int stats_impl(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes, const peer_dst * publish)
{
	int st = check_train_args("nnf_bn_train_stats", n, c, hw);
	if (st != NNF_OK)
		return st;
	if (!sums || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_stats: null pointer");
	if (!workspace || workspace_bytes < nnf_bn_train_workspace_bytes(n, c, hw) || (reinterpret_cast<uintptr_t>(workspace) & 7))
		return set_error(NNF_ERR_WORKSPACE, "nnf_bn_train_stats: workspace of %zu bytes (8-byte aligned) required, got %zu", nnf_bn_train_workspace_bytes(n, c, hw), workspace_bytes);
	chan_geom g;
	group_geom gg;
	cudaStream_t s = (cudaStream_t)stream;
	if (make_group_geom(gg, n, c, hw, aligned16(x)))
	{
		if (gg.vectors_per_thread == 1)
			bn_stats_grouped_kernel<1><<<gg.groups * gg.split, kThreads, 0, s>>>(static_cast<double *>(workspace), x, gg);
		else
			bn_stats_grouped_kernel<2><<<gg.groups * gg.split, kThreads, 0, s>>>(static_cast<double *>(workspace), x, gg);
		st = check_launch("bn_stats_grouped_kernel");
		g.c = gg.c;
		g.split = gg.split;
	}
	else
	{
		st = make_chan_geom(g, "nnf_bn_train_stats", n, c, hw, aligned16(x), resident_ctas_per_sm(bn_stats_kernel), 1);
		if (st != NNF_OK)
			return st;
		bn_stats_kernel<<<g.c * g.split, kThreads, 0, s>>>(static_cast<double *>(workspace), x, g);
		st = check_launch("bn_stats_kernel");
	}
	if (st != NNF_OK)
		return st;
	if (publish)
	{
		bn_reduce_publish_kernel<<<1, 1024, 0, s>>>(sums, static_cast<const double *>(workspace), g.c, g.split, 2, nullptr, 0, *publish, 2);
		return check_launch("bn_reduce_publish_kernel");
	}
	bn_reduce_partials_kernel<<<(unsigned)div_up(c, 128), 128, 0, s>>>(sums, static_cast<const double *>(workspace), g.c, g.split, 2, 0);
	return check_launch("bn_reduce_partials_kernel");
}
}

namespace
{
	int apply_impl(nnf_stream_t stream, float * y, float * saved, const float * x, const float * gamma, const float * beta, const float * sums,
		const peer_src * peer, double count_total, float eps, const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw);

	int make_peer_src(peer_src& s, const void * my_buf, int world, int k, int kmax, uint32_t seq, const char * who)
	{
		if (world < 1 || world > kMaxRanks || kmax < k || !my_buf || seq == 0)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: bad peer arguments (world %d, %d floats, slots of %d)", who, world, k, kmax);
		s.mine = static_cast<const float *>(my_buf); s.world = world; s.kmax = kmax; s.seq = seq; s.error = device_error_word();
		return NNF_OK;
	}
}

extern "C" int nnf_bn_train_apply_act_peer(nnf_stream_t stream, float * y, float * saved, const float * x,
	const float * gamma, const float * beta, const void * my_buf, int world, int kmax, uint32_t seq, double count_total, float eps,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw)
{
	peer_src src;
	int st = make_peer_src(src, my_buf, world, (int)(2 * c), kmax, seq, "nnf_bn_train_apply_act_peer");
	if (st != NNF_OK)
		return st;
	return apply_impl(stream, y, saved, x, gamma, beta, nullptr, &src, count_total, eps, acts, n_acts, n, c, hw);
}

extern "C" int nnf_bn_train_apply_act(nnf_stream_t stream, float * y, float * saved, const float * x,
	const float * gamma, const float * beta, const float * sums, double count_total, float eps,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw)
{
	return apply_impl(stream, y, saved, x, gamma, beta, sums, nullptr, count_total, eps, acts, n_acts, n, c, hw);
}

namespace
{
int apply_impl(nnf_stream_t stream, float * y, float * saved, const float * x, const float * gamma, const float * beta, const float * sums,
	const peer_src * peer, double count_total, float eps, const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw)
{
	int st = check_train_args("nnf_bn_train_apply_act", n, c, hw);
	if (st != NNF_OK)
		return st;
	if (!y || !x || !gamma || !beta || (!sums && !peer))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_apply_act: null pointer");
	if (!(count_total >= 1.0))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_apply_act: count_total = %g", count_total);
	act_chain chain;
	st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	int prelus = 0;
	for (int i = 0; i < chain.n; ++i)
		prelus += chain.a[i].kind == NNF_ACT_PRELU;
	group_geom gg;
	if (!peer && prelus <= 1 && make_group_geom(gg, n, c, hw, aligned16(x) && aligned16(y)))
	{
		apply_params p = {};
		p.y = y; p.x = x; p.gamma = gamma; p.beta = beta; p.sums = sums; p.saved = saved; p.count_total = count_total; p.eps = eps;
		p.chain = chain;
		const unsigned grid = gg.groups * gg.split;
		cudaStream_t s = (cudaStream_t)stream;
		#define NNF_GROUPED_APPLY(A0, A1) \
			do { if (gg.vectors_per_thread == 1) bn_apply_grouped_kernel<A0, A1, 1><<<grid, kThreads, 0, s>>>(p, gg); \
			     else bn_apply_grouped_kernel<A0, A1, 2><<<grid, kThreads, 0, s>>>(p, gg); } while (0)
		switch (chain_id(chain))
		{
		case 0: NNF_GROUPED_APPLY(NNF_ACT_NONE, 0); break;
		case 1: NNF_GROUPED_APPLY(NNF_ACT_PRELU, NNF_ACT_ELU); break;
		case 2: NNF_GROUPED_APPLY(NNF_ACT_RELU, 0); break;
		default: NNF_GROUPED_APPLY(-1, 0); break;
		}
		#undef NNF_GROUPED_APPLY
		return check_launch("bn_apply_grouped_kernel");
	}
	// planes large enough to keep a CTA busy and whole float4s: the channel-ordered kernel (L2 reuse after the
	// statistics kernel); anything else: the flat streaming kernel
	if (hw % 4 == 0 && (n * hw >= 16384 || peer) && prelus <= 1 && aligned16(x) && aligned16(y) && n * hw <= kMaxElemsPerLaunch && tune().apply_flat != 1)
	{
		chan_geom g;
		st = make_chan_geom(g, "nnf_bn_train_apply_act", n, c, hw, true, resident_ctas_per_sm(bn_apply_channel_kernel<-1, 0>), 8);
		if (st != NNF_OK)
			return st;
		apply_params p = {};
		p.y = y; p.x = x; p.gamma = gamma; p.beta = beta; p.sums = sums; p.saved = saved; p.count_total = count_total; p.eps = eps;
		p.chain = chain;
		if (peer)
			p.peer = *peer;
		cudaStream_t s = (cudaStream_t)stream;
		switch (chain_id(chain))
		{
		case 0: bn_apply_channel_kernel<NNF_ACT_NONE, 0><<<g.c * g.split, kThreads, 0, s>>>(p, g); break;
		case 1: bn_apply_channel_kernel<NNF_ACT_PRELU, NNF_ACT_ELU><<<g.c * g.split, kThreads, 0, s>>>(p, g); break;
		case 2: bn_apply_channel_kernel<NNF_ACT_RELU, 0><<<g.c * g.split, kThreads, 0, s>>>(p, g); break;
		default: bn_apply_channel_kernel<-1, 0><<<g.c * g.split, kThreads, 0, s>>>(p, g); break;
		}
		return check_launch("bn_apply_channel_kernel");
	}
	if (peer)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_apply_act_peer: this shape runs the flat kernel, which reads a plain sums buffer; use nnf_peer_exchange_sum + nnf_bn_train_apply_act");
	bn_source bn = {};
	bn.gamma = gamma; bn.beta = beta; bn.sums = sums; bn.saved = saved; bn.count_total = count_total; bn.eps = eps;
	return run_elementwise((cudaStream_t)stream, y, x, nullptr, 1.0F, bn, chain, n, c, hw);
}
}

namespace
{
	int fill_bwd(bwd_params& p, const char * who, const float * dy, const float * x, const float * gamma, const float * beta, const float * saved,
		const nnf_act * acts, int n_acts)
	{
		if (!dy || !x || !gamma || !beta || !saved)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
		int st = make_chain(p.chain, acts, n_acts, true);
		if (st != NNF_OK)
			return st;
		chain_fill_backward_constants(p.chain, acts, n_acts);
		int prelus = 0;
		for (int i = 0; i < p.chain.n; ++i)
			prelus += p.chain.a[i].kind == NNF_ACT_PRELU;
		if (prelus > 1)
			return set_error(NNF_ERR_UNSUPPORTED, "%s: at most one PReLU per fused chain", who);
		p.dy = dy; p.x = x; p.gamma = gamma; p.beta = beta; p.saved = saved;
		return NNF_OK;
	}
}

namespace
{
	int bwd_stats_impl(nnf_stream_t stream, float * bsums, float * gsums, const float * dy, const float * x,
		const float * gamma, const float * beta, const float * saved, const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
		void * workspace, size_t workspace_bytes, const peer_dst * publish);
}

extern "C" int nnf_bn_train_bwd_stats(nnf_stream_t stream, float * bsums, float * gsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes)
{
	return bwd_stats_impl(stream, bsums, gsums, dy, x, gamma, beta, saved, acts, n_acts, n, c, hw, workspace, workspace_bytes, nullptr);
}

extern "C" int nnf_bn_train_bwd_stats_publish(nnf_stream_t stream, float * bsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes, void * const * peer_bufs, int rank, int world, int kmax, uint32_t seq)
{
	peer_dst d;
	int st = make_peer_dst(d, peer_bufs, rank, world, (int)(2 * c), kmax, seq, "nnf_bn_train_bwd_stats_publish");
	if (st != NNF_OK)
		return st;
	return bwd_stats_impl(stream, bsums, nullptr, dy, x, gamma, beta, saved, acts, n_acts, n, c, hw, workspace, workspace_bytes, &d);
}

namespace
{
int bwd_stats_impl(nnf_stream_t stream, float * bsums, float * gsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved, const nnf_act * acts, int n_acts, int64_t n, int64_t c, int64_t hw,
	void * workspace, size_t workspace_bytes, const peer_dst * publish)
{
	int st = check_train_args("nnf_bn_train_bwd_stats", n, c, hw);
	if (st != NNF_OK)
		return st;
	if (!bsums)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_stats: null pointer");
	if (!workspace || workspace_bytes < nnf_bn_train_workspace_bytes(n, c, hw) || (reinterpret_cast<uintptr_t>(workspace) & 7))
		return set_error(NNF_ERR_WORKSPACE, "nnf_bn_train_bwd_stats: workspace of %zu bytes (8-byte aligned) required, got %zu", nnf_bn_train_workspace_bytes(n, c, hw), workspace_bytes);
	bwd_params p = {};
	st = fill_bwd(p, "nnf_bn_train_bwd_stats", dy, x, gamma, beta, saved, acts, n_acts);
	if (st != NNF_OK)
		return st;
	chan_geom g;
	group_geom gg;
	cudaStream_t s = (cudaStream_t)stream;
	if (make_group_geom(gg, n, c, hw, aligned16(x) && aligned16(dy)))
	{
		double * ws = static_cast<double *>(workspace);
		const unsigned grid = gg.groups * gg.split;
		#define NNF_GROUPED_BWD_STATS(A0, A1) \
			do { if (gg.vectors_per_thread == 1) bn_bwd_stats_grouped_kernel<A0, A1, 1><<<grid, kThreads, 0, s>>>(ws, p, gg); \
			     else bn_bwd_stats_grouped_kernel<A0, A1, 2><<<grid, kThreads, 0, s>>>(ws, p, gg); } while (0)
		switch (chain_id(p.chain))
		{
		case 0: NNF_GROUPED_BWD_STATS(NNF_ACT_NONE, 0); break;
		case 1: NNF_GROUPED_BWD_STATS(NNF_ACT_PRELU, NNF_ACT_ELU); break;
		case 2: NNF_GROUPED_BWD_STATS(NNF_ACT_RELU, 0); break;
		default: NNF_GROUPED_BWD_STATS(-1, 0); break;
		}
		#undef NNF_GROUPED_BWD_STATS
		st = check_launch("bn_bwd_stats_grouped_kernel");
		g.c = gg.c;
		g.split = gg.split;
	}
	else
	{
		st = make_chan_geom(g, "nnf_bn_train_bwd_stats", n, c, hw, aligned16(x) && aligned16(dy), resident_ctas_per_sm(bn_bwd_stats_kernel<-1, 0>), 2);
		if (st != NNF_OK)
			return st;
		switch (chain_id(p.chain))
		{
		case 0: bn_bwd_stats_kernel<NNF_ACT_NONE, 0><<<g.c * g.split, kThreads, 0, s>>>(static_cast<double *>(workspace), p, g); break;
		case 1: bn_bwd_stats_kernel<NNF_ACT_PRELU, NNF_ACT_ELU><<<g.c * g.split, kThreads, 0, s>>>(static_cast<double *>(workspace), p, g); break;
		case 2: bn_bwd_stats_kernel<NNF_ACT_RELU, 0><<<g.c * g.split, kThreads, 0, s>>>(static_cast<double *>(workspace), p, g); break;
		default: bn_bwd_stats_kernel<-1, 0><<<g.c * g.split, kThreads, 0, s>>>(static_cast<double *>(workspace), p, g); break;
		}
		st = check_launch("bn_bwd_stats_kernel");
	}
	if (st != NNF_OK)
		return st;
	if (publish)
	{
		bn_reduce_publish_kernel<<<1, 1024, 0, s>>>(bsums, static_cast<const double *>(workspace), g.c, g.split, 3, gsums, 2, *publish, 2);
		return check_launch("bn_reduce_publish_kernel");
	}
	bn_reduce_partials_kernel<<<(unsigned)div_up(c, 128), 128, 0, s>>>(bsums, static_cast<const double *>(workspace), g.c, g.split, 3, 0, gsums, 2);
	return check_launch("bn_reduce_partials_kernel");
}
}

namespace
{
	int bwd_apply_impl(nnf_stream_t stream, float * dx, const float * dy, const float * x,
		const float * gamma, const float * beta, const float * saved,
		const float * gsums, const peer_src * peer, const float * bsums, double count_total,
		const nnf_act * acts, int n_acts,
		float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
		const float * mean, const float * invsigma, float entry_count,
		int64_t n, int64_t c, int64_t hw, int add_to_destination);
}

extern "C" int nnf_bn_train_bwd_apply(nnf_stream_t stream, float * dx, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const float * gsums, const float * bsums, double count_total,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	return bwd_apply_impl(stream, dx, dy, x, gamma, beta, saved, gsums, nullptr, bsums, count_total, acts, n_acts,
		grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope, mean, invsigma, entry_count, n, c, hw, add_to_destination);
}

extern "C" int nnf_bn_train_bwd_apply_peer(nnf_stream_t stream, float * dx, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const void * my_buf, int world, int kmax, uint32_t seq, const float * bsums, double count_total,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	peer_src src;
	int st = make_peer_src(src, my_buf, world, (int)(2 * c), kmax, seq, "nnf_bn_train_bwd_apply_peer");
	if (st != NNF_OK)
		return st;
	return bwd_apply_impl(stream, dx, dy, x, gamma, beta, saved, nullptr, &src, bsums, count_total, acts, n_acts,
		grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope, mean, invsigma, entry_count, n, c, hw, add_to_destination);
}

namespace
{
int bwd_apply_impl(nnf_stream_t stream, float * dx, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved,
	const float * gsums, const peer_src * peer, const float * bsums, double count_total,
	const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	int st = check_train_args("nnf_bn_train_bwd_apply", n, c, hw);
	if (st != NNF_OK)
		return st;
	if (!dx || (!gsums && !peer))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_apply: null pointer");
	if ((grad_gamma || grad_beta || grad_slope) && !bsums)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_apply: per-channel gradients requested without the local sums");
	if ((grad_mean && !mean) || (grad_invsigma && !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_apply: running-statistics gradients requested without the running statistics");
	if (!(count_total >= 1.0))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_apply: count_total = %g", count_total);
	bwd_params p = {};
	st = fill_bwd(p, "nnf_bn_train_bwd_apply", dy, x, gamma, beta, saved, acts, n_acts);
	if (st != NNF_OK)
		return st;
	p.dx = dx; p.gsums = gsums; p.bsums = bsums; p.count_total = count_total;
	if (peer)
		p.peer = *peer;
	p.grad_gamma = grad_gamma; p.grad_beta = grad_beta; p.grad_mean = grad_mean; p.grad_invsigma = grad_invsigma; p.grad_slope = grad_slope;
	p.mean = mean; p.invsigma = invsigma; p.entry_count = entry_count;
	p.add = add_to_destination ? 1 : 0;
	group_geom gg;
	if (!peer && make_group_geom(gg, n, c, hw, aligned16(x) && aligned16(dy) && aligned16(dx)))
	{
		const unsigned grid = gg.groups * gg.split;
		cudaStream_t s = (cudaStream_t)stream;
		#define NNF_GROUPED_BWD_APPLY(A0, A1) \
			do { if (gg.vectors_per_thread == 1) bn_bwd_apply_grouped_kernel<A0, A1, 1><<<grid, kThreads, 0, s>>>(p, gg); \
			     else bn_bwd_apply_grouped_kernel<A0, A1, 2><<<grid, kThreads, 0, s>>>(p, gg); } while (0)
		switch (chain_id(p.chain))
		{
		case 0: NNF_GROUPED_BWD_APPLY(NNF_ACT_NONE, 0); break;
		case 1: NNF_GROUPED_BWD_APPLY(NNF_ACT_PRELU, NNF_ACT_ELU); break;
		case 2: NNF_GROUPED_BWD_APPLY(NNF_ACT_RELU, 0); break;
		default: NNF_GROUPED_BWD_APPLY(-1, 0); break;
		}
		#undef NNF_GROUPED_BWD_APPLY
		return check_launch("bn_bwd_apply_grouped_kernel");
	}
	chan_geom g;
	st = make_chan_geom(g, "nnf_bn_train_bwd_apply", n, c, hw, aligned16(x) && aligned16(dy) && aligned16(dx), resident_ctas_per_sm(bn_bwd_apply_kernel<-1, 0>), 8);
	if (st != NNF_OK)
		return st;
	switch (chain_id(p.chain))
	{
	case 0: bn_bwd_apply_kernel<NNF_ACT_NONE, 0><<<g.c * g.split, kThreads, 0, (cudaStream_t)stream>>>(p, g); break;
	case 1: bn_bwd_apply_kernel<NNF_ACT_PRELU, NNF_ACT_ELU><<<g.c * g.split, kThreads, 0, (cudaStream_t)stream>>>(p, g); break;
	case 2: bn_bwd_apply_kernel<NNF_ACT_RELU, 0><<<g.c * g.split, kThreads, 0, (cudaStream_t)stream>>>(p, g); break;
	default: bn_bwd_apply_kernel<-1, 0><<<g.c * g.split, kThreads, 0, (cudaStream_t)stream>>>(p, g); break;
	}
	return check_launch("bn_bwd_apply_kernel");
}
}

extern "C" size_t nnf_prelu_bwd_weights_workspace_bytes(int64_t n, int64_t c, int64_t hw)
{
	return nnf_bn_train_workspace_bytes(n, c, hw);
}

extern "C" int nnf_prelu_bwd_weights(nnf_stream_t stream, float * dslope, const float * dy, const float * x,
	int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes)
{
	if (n < 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_prelu_bwd_weights: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (n == 0)
		return NNF_OK;
	if (!dslope || !dy || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_prelu_bwd_weights: null pointer");
	if (!workspace || workspace_bytes < nnf_prelu_bwd_weights_workspace_bytes(n, c, hw) || (reinterpret_cast<uintptr_t>(workspace) & 7))
		return set_error(NNF_ERR_WORKSPACE, "nnf_prelu_bwd_weights: workspace of %zu bytes (8-byte aligned) required, got %zu", nnf_prelu_bwd_weights_workspace_bytes(n, c, hw), workspace_bytes);
	chan_geom g;
	group_geom gg;
	int st;
	cudaStream_t s = (cudaStream_t)stream;
	if (make_group_geom(gg, n, c, hw, aligned16(x) && aligned16(dy)))
	{
		if (gg.vectors_per_thread == 1)
			prelu_dslope_grouped_kernel<1><<<gg.groups * gg.split, kThreads, 0, s>>>(static_cast<double *>(workspace), dy, x, gg);
		else
			prelu_dslope_grouped_kernel<2><<<gg.groups * gg.split, kThreads, 0, s>>>(static_cast<double *>(workspace), dy, x, gg);
		st = check_launch("prelu_dslope_grouped_kernel");
		g.c = gg.c;
		g.split = gg.split;
	}
	else
	{
		st = make_chan_geom(g, "nnf_prelu_bwd_weights", n, c, hw, aligned16(x) && aligned16(dy), resident_ctas_per_sm(prelu_dslope_kernel), 1);
		if (st != NNF_OK)
			return st;
		prelu_dslope_kernel<<<g.c * g.split, kThreads, 0, s>>>(static_cast<double *>(workspace), dy, x, g);
		st = check_launch("prelu_dslope_kernel");
	}
	if (st != NNF_OK)
		return st;
	bn_reduce_partials_kernel<<<(unsigned)div_up(c, 128), 128, 0, s>>>(dslope, static_cast<const double *>(workspace), g.c, g.split, 1, 1);
	return check_launch("bn_reduce_partials_kernel");
}

// ---------------------------------------------------------------------------------------------
// Batch statistics for callers that have no workspace to hand over.
//
// Some hosts of this library may not allocate device memory at the point where they call it: an
// nnForge layer object is only ever given the buffers the scheduler planned up front from the
// layer's own size answers (and the stock batch-norm updater asks for no working buffer, so a
// drop-in that must keep those answers has nowhere to get one); the scheduler also measures free
// memory once and then fills it, so a later cudaMalloc can fail or stall every stream of the device.
// For them the per-CTA partial sums live in the fixed array below, which every GPU that loads the
// library holds until the process exits.
//
// Limit: kStaticMaxChannels channels (the array is kStaticMaxChannels * kMaxSplit * kSums doubles =
// 1.5 MiB). The array is shared by all calls on a device and keeps whatever the last call left in
// it; nothing in it has to start at zero, because every slot the reduce kernel reads is written by
// the statistics kernel of the same call first. Two calls that overlap on one GPU (different
// streams) would race on it.
constexpr int kStaticMaxChannels = 1024;
static __device__ __align__(256) double nnf_static_stats_scratch[size_t(kStaticMaxChannels) * nnf::kMaxSplit * nnf::kSums];

namespace
{
	constexpr int kStaticMaxDevices = 64;
	double * g_static_scratch_address[kStaticMaxDevices] = {};
	std::mutex g_static_scratch_mutex;

	// In host code the array's name is only a handle; the device address has to be asked for, once per
	// device, with that device current.
	int static_scratch_for_current_device(double *& address)
	{
		int device = -1;
		cudaError_t e = cudaGetDevice(&device);
		if (e != cudaSuccess)
			return set_error(NNF_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
		if (device < 0 || device >= kStaticMaxDevices)
			return set_error(NNF_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range 0..%d", device, kStaticMaxDevices - 1);
		std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
		if (!g_static_scratch_address[device])
		{
			double * p = nullptr;
			e = cudaGetSymbolAddress((void **)&p, nnf_static_stats_scratch);
			if (e != cudaSuccess || !p)
				return set_error(NNF_ERR_CUDA, "cudaGetSymbolAddress(static statistics scratch): %s", cudaGetErrorString(e));
			g_static_scratch_address[device] = p;
		}
		address = g_static_scratch_address[device];
		return NNF_OK;
	}
}

extern "C" int nnf_bn_train_stats_static(nnf_stream_t stream, float * sums, const float * x, int64_t n, int64_t c, int64_t hw)
{
	int st = check_train_args("nnf_bn_train_stats_static", n, c, hw);
	if (st != NNF_OK)
		return st;
	if (c > kStaticMaxChannels)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_stats_static: %lld channels exceed the built-in scratch, which holds at most %d; "
			"use nnf_bn_train_stats with a workspace instead", (long long)c, kStaticMaxChannels);
	if (!sums || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_stats_static: null pointer");
	chan_geom g;
	st = make_chan_geom(g, "nnf_bn_train_stats_static", n, c, hw, aligned16(x), resident_ctas_per_sm(bn_stats_kernel), 1);
	if (st != NNF_OK)
		return st;
	double * scratch = nullptr;
	st = static_scratch_for_current_device(scratch);
	if (st != NNF_OK)
		return st;
	cudaStream_t s = (cudaStream_t)stream;
	bn_stats_kernel<<<g.c * g.split, kThreads, 0, s>>>(scratch, x, g);
	st = check_launch("bn_stats_kernel");
	if (st != NNF_OK)
		return st;
	bn_reduce_partials_kernel<<<(unsigned)div_up(c, 128), 128, 0, s>>>(sums, scratch, g.c, g.split, 2, 0);
	return check_launch("bn_reduce_partials_kernel");
}
