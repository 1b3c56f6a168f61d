// Training batch norm + activation chain, forward and backward, reading every input ONCE: a CTA pulls one PIECE of a
// channel (a slice of entries, about 50 KB of x, or of x and dy) into shared memory with bulk asynchronous copies,
// adds the piece's statistics, publishes them, waits until the other pieces of the channel have done the same, and
// then normalises its piece straight out of shared memory. HBM and the SMs see 8 (forward) / 12 (backward) bytes per
// element; the forms that read twice move 12 / 20 through the SMs even when the second read hits L2.
//
// Why the wait cannot hang: a CTA takes a ticket when it STARTS and serves item number ticket, items are numbered
// channel by channel, so the pieces of a channel hold consecutive tickets. Consider the lowest channel that is not
// complete. Everything with a smaller ticket than its pieces has finished, and every CTA that has started holds a
// smaller ticket than any CTA that has not; so the CTAs that occupy the machine while one of that channel's pieces
// has not started yet are all pieces of that same channel - at most pieces-1 of them. The plan therefore only accepts
// shapes for which the machine holds at least `pieces` CTAs of this kernel at once (checked with the occupancy query),
// and then a free slot always exists for the missing piece. Every wait is bounded all the same and reports through
// the word read by nnf_fused_error_check (value 4: sibling pieces, value 1: the bulk copies).
//
// Unlike the cluster form of the same idea (nnf_bn_fused.cu) nothing here needs co-scheduled CTAs: pieces are
// ordinary CTAs, four per SM, and an SM always has pieces in different phases - some loading, some storing.
#include "nnf_async.cuh"

#include <stdlib.h>

namespace nnf
{
	namespace
	{
		constexpr int kResThreads = 256;
		constexpr int kResMaxPieces = 64;               // pieces per channel (sizes the partial sums like the other forms)
		constexpr uint32_t kResPollLimit = 1u << 22;    // rounds of the wait for the sibling pieces (about half a microsecond each)

		struct resident_params
		{
			const float * x;
			const float * dy;        // backward only
			float * out;             // y (forward) or dx (backward)
			const float * gamma;
			const float * beta;
			float * saved;           // forward: written {mean, invstd}; backward: read
			float * sums;            // forward: {sum x, sum x^2} (may be null); backward: bsums[3C]
			float * grad_gamma, * grad_beta, * grad_mean, * grad_invsigma, * grad_slope;
			const float * mean, * invsigma;
			float entry_count;
			act_chain chain;
			uint32_t n, c, hw;
			uint32_t entries, pieces;   // entries per piece, pieces per channel
			uint32_t piece_floats;      // floats of one tensor's piece in shared memory
			uint32_t total_items;
			fastdiv d_pieces, d_vpp;
			double count;
			float eps;
			double * partial;           // [c][pieces][3]
			uint32_t * done;            // [c], zero at kernel start
			uint32_t * ticket;          // zero at kernel start
			int * error;
		};

		__device__ __forceinline__ uint32_t res_ld_acquire(const uint32_t * p)
		{
			uint32_t v;
			asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
			return v;
		}

		__device__ __forceinline__ double res_warp_sum(double v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			return v;
		}

		template <int A0, int A1, bool BWD>
		__global__ void __launch_bounds__(kResThreads) bn_train_resident_kernel(const resident_params p)
		{
			constexpr int K = BWD ? 3 : 2;
			extern __shared__ __align__(128) unsigned char s_dyn[];
			float * sx = reinterpret_cast<float *>(s_dyn);
			float * sd = sx + p.piece_floats;
			__shared__ __align__(8) uint64_t s_bar;
			__shared__ double s_red[(kResThreads / 32) * K];
			__shared__ uint32_t s_item;
			__shared__ float s_tot[2];

			if (threadIdx.x == 0)
			{
				s_item = atomicAdd(p.ticket, 1u);
				mbar_init(&s_bar, 1);
				asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
			}
			__syncthreads();
			const uint32_t item = s_item;
			if (item >= p.total_items)
				return;
			const uint32_t walk = p.d_pieces.div(item);
			const uint32_t sp = item - walk * p.pieces;
			// the backward launch walks the channels downwards: the forward launch, which walks upwards, left the highest in L2
			const uint32_t ch = BWD ? p.c - 1 - walk : walk;
			const uint32_t e0 = sp * p.entries;
			const uint32_t e1 = min(e0 + p.entries, p.n);
			const uint32_t np = e1 > e0 ? e1 - e0 : 0;
			const uint32_t plane_bytes = p.hw * 4;
			const uint32_t vpp = p.hw >> 2;
			const uint32_t nvec = np * vpp;

			// ---- the piece comes into shared memory: one bulk copy per plane and tensor -----------------------------
			if (threadIdx.x < 32)
			{
				if (threadIdx.x == 0)
					mbar_expect_tx(&s_bar, np * plane_bytes * (BWD ? 2u : 1u));
				__syncwarp();
				for (uint32_t pl = threadIdx.x; pl < np; pl += 32)
				{
					const size_t off = (size_t(e0 + pl) * p.c + ch) * p.hw;
					bulk_load(sx + size_t(pl) * p.hw, p.x + off, plane_bytes, &s_bar);
					if (BWD)
						bulk_load(sd + size_t(pl) * p.hw, p.dy + off, plane_bytes, &s_bar);
				}
			}
			const float slope = chain_slope(p.chain, ch);
			float mean = 0.0F, invstd = 0.0F, mult = 0.0F, add = 0.0F;
			if (BWD)
			{
				mean = __ldg(p.saved + ch);
				invstd = __ldg(p.saved + p.c + ch);
				mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
				add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
			}
			if (!mbar_wait(&s_bar, 0) && p.error)
				*p.error = 1;

			// ---- this piece's statistics --------------------------------------------------------------------------------
			const float4 * sx4 = reinterpret_cast<const float4 *>(sx);
			const float4 * sd4 = reinterpret_cast<const float4 *>(sd);
			double acc[K];
			if (!BWD)
			{
				float s = 0.0F, q = 0.0F;
				for (uint32_t i = threadIdx.x; i < nvec; i += kResThreads)
				{
					const float4 a = sx4[i];
					s += (a.x + a.y) + (a.z + a.w);
					q = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, q))));
				}
				acc[0] = double(s);
				acc[1] = double(q);
			}
			else
			{
				float sb = 0.0F, sg = 0.0F, ss = 0.0F;
				auto element = [&](float x, float dy)
				{
					const float u = __fadd_rn(__fmul_rn(x, mult), add);
					float term;
					const float du = chain_backward<A0, A1>(p.chain, u, dy, slope, term);
					const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
					sb += du;
					sg = fmaf(du, xhat, sg);
					ss += term;
				};
				for (uint32_t i = threadIdx.x; i < nvec; i += kResThreads)
				{
					const float4 a = sx4[i], d = sd4[i];
					element(a.x, d.x); element(a.y, d.y); element(a.z, d.z); element(a.w, d.w);
				}
				acc[0] = double(sb);
				acc[1] = double(sg);
				acc[K - 1] = double(ss);
			}
			{
				const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
				#pragma unroll
				for (int k = 0; k < K; ++k)
					acc[k] = res_warp_sum(acc[k]);
				if (lane == 0)
				{
					#pragma unroll
					for (int k = 0; k < K; ++k)
						s_red[w * K + k] = acc[k];
				}
			}
			__syncthreads();
			if (threadIdx.x == 0)
			{
				double * out = p.partial + (size_t(ch) * p.pieces + sp) * 3;
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					double t = 0.0;
					for (int i = 0; i < kResThreads / 32; ++i)
						t += s_red[i * K + k];
					out[k] = t;
				}
				__threadfence(); // the partial sums are visible before the count
				atomicAdd(p.done + ch, 1u);
				// ---- wait (bounded) for the sibling pieces ------------------------------------------------------------
				bool ready = false;
				for (uint32_t round = 0; round < kResPollLimit; ++round)
				{
					if (res_ld_acquire(p.done + ch) >= p.pieces)
					{
						ready = true;
						break;
					}
					__nanosleep(100);
				}
				if (!ready && p.error)
					*p.error = 4;
			}
			__syncthreads();
			if (threadIdx.x < 32)
			{
				// all pieces' partial sums in piece order: lane l takes pieces l and l + 32, then a fixed shuffle tree
				double tot[K];
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					double t = 0.0;
					for (uint32_t q = threadIdx.x; q < p.pieces; q += 32)
						t += __ldcg(p.partial + (size_t(ch) * p.pieces + q) * 3 + k);
					tot[k] = res_warp_sum(t);
				}
				if (threadIdx.x == 0)
				{
					if (!BWD)
					{
						const double m = tot[0] / p.count;
						double var = tot[1] / p.count - m * m;
						var = var < 0.0 ? 0.0 : var;
						const float fmean = float(m);
						const float finv = float(1.0 / sqrt(var + double(p.eps)));
						s_tot[0] = fmean;
						s_tot[1] = finv;
						if (sp == 0)
						{
							p.saved[ch] = fmean;
							p.saved[p.c + ch] = finv;
							if (p.sums)
							{
								p.sums[ch] = float(tot[0]);
								p.sums[p.c + ch] = float(tot[1]);
							}
						}
					}
					else
					{
						const float fb = float(tot[0]), fg = float(tot[1]), fs = float(tot[K - 1]);
						// the same float-rounded sums the two-kernel form passes between its kernels
						s_tot[0] = float(double(fb) / p.count);
						s_tot[1] = float(double(fg) / p.count);
						if (sp == 0)
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
					}
				}
			}
			__syncthreads();

			// ---- normalise the piece out of shared memory ----------------------------------------------------------------
			const size_t entry_stride = size_t(p.c) * p.hw;
			float * out0 = p.out + (size_t(e0) * p.c + ch) * p.hw;
			if (!BWD)
			{
				const float fmean = s_tot[0], finv = s_tot[1];
				const float fmult = __fmul_rn(__ldg(p.gamma + ch), finv);
				const float fadd = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(fmult, fmean));
				for (uint32_t i = threadIdx.x; i < nvec; i += kResThreads)
				{
					const float4 a = sx4[i];
					const uint32_t pl = p.d_vpp.div(i);
					float4 o;
					o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.x, fmult), fadd), slope);
					o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.y, fmult), fadd), slope);
					o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.z, fmult), fadd), slope);
					o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a.w, fmult), fadd), slope);
					st_stream(reinterpret_cast<float4 *>(out0 + pl * entry_stride) + (i - pl * vpp), o);
				}
			}
			else
			{
				const float c2 = s_tot[0], c3 = s_tot[1];
				auto element = [&](float x, float dy) -> float
				{
					const float u = __fadd_rn(__fmul_rn(x, mult), add);
					float term;
					const float du = chain_backward<A0, A1>(p.chain, u, dy, slope, term);
					const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
					return mult * ((du - c2) - xhat * c3);
				};
				for (uint32_t i = threadIdx.x; i < nvec; i += kResThreads)
				{
					const float4 a = sx4[i], d = sd4[i];
					const uint32_t pl = p.d_vpp.div(i);
					st_stream(reinterpret_cast<float4 *>(out0 + pl * entry_stride) + (i - pl * vpp),
						make_float4(element(a.x, d.x), element(a.y, d.y), element(a.z, d.z), element(a.w, d.w)));
				}
			}
		}

		int res_env(const char * name, int fallback)
		{
			const char * v = getenv(name);
			return v ? atoi(v) : fallback;
		}

		// Piece size: NNF_RES_PIECE_KB (tuning aid) kilobytes of shared memory per CTA, four CTAs per SM by default.
		template <class Kernel>
		bool plan_resident(resident_params& p, size_t& smem, Kernel kernel, int64_t n, int64_t c, int64_t hw, int tensors)
		{
			if (hw % 4 != 0 || n < 1 || c < 1 || n >= (int64_t(1) << 31) || hw >= (int64_t(1) << 24) || c >= (int64_t(1) << 24))
				return false;
			const int64_t entry_bytes = hw * 4 * tensors;
			const int64_t budget = int64_t(res_env("NNF_RES_PIECE_KB", 52)) * 1024;
			int64_t emax = budget / entry_bytes;
			if (emax < 1) emax = 1;
			if (emax > n) emax = n;
			if (div_up(n, emax) > kResMaxPieces)
				emax = div_up(n, kResMaxPieces);
			// among piece sizes down to three quarters of the largest, the one that wastes the fewest entries in the last piece
			int64_t best = emax, best_waste = div_up(n, emax) * emax - n;
			for (int64_t e = emax - 1; e >= 1 && e * 4 >= emax * 3 && div_up(n, e) <= kResMaxPieces; --e)
			{
				const int64_t waste = div_up(n, e) * e - n;
				if (waste < best_waste)
				{
					best = e;
					best_waste = waste;
				}
			}
			const int64_t entries = best, pieces = div_up(n, entries);
			smem = size_t(entries) * entry_bytes;
			if (smem > 200 * 1024 || c * pieces >= (int64_t(1) << 31))
				return false;
			if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
			{
				cudaGetLastError();
				return false;
			}
			int per_sm = 0;
			if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kResThreads, smem) != cudaSuccess || per_sm < 1)
			{
				cudaGetLastError();
				return false;
			}
			int device = 0, sms = 0;
			if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
			{
				cudaGetLastError();
				return false;
			}
			if (int64_t(sms) * per_sm < pieces)
				return false; // the pieces of one channel must be able to be resident together (see the head of this file)
			p.n = (uint32_t)n; p.c = (uint32_t)c; p.hw = (uint32_t)hw;
			p.entries = (uint32_t)entries;
			p.pieces = (uint32_t)pieces;
			p.piece_floats = (uint32_t)(entries * hw);
			p.total_items = (uint32_t)(c * pieces);
			p.d_pieces = fastdiv(p.pieces);
			p.d_vpp = fastdiv((uint32_t)(hw / 4));
			p.count = double(n) * double(hw);
			return true;
		}

		template <class Kernel>
		int launch_resident(Kernel kernel, resident_params& p, size_t smem, void * workspace, size_t workspace_bytes, cudaStream_t s, const char * what)
		{
			const size_t need = size_t(p.c) * p.pieces * 3 * sizeof(double) + (size_t(p.c) + 1) * sizeof(uint32_t);
			if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 7) || workspace_bytes < need)
				return 1;
			p.partial = static_cast<double *>(workspace);
			p.done = reinterpret_cast<uint32_t *>(p.partial + size_t(p.c) * p.pieces * 3);
			p.ticket = p.done + p.c;
			p.error = device_error_word();
			cudaError_t e = cudaMemsetAsync(p.done, 0, (size_t(p.c) + 1) * sizeof(uint32_t), s);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s: cudaMemsetAsync: %s", what, cudaGetErrorString(e));
			kernel<<<p.total_items, kResThreads, smem, s>>>(p);
			return check_launch(what);
		}

		template <bool BWD>
		int resident_impl(resident_params& p, const act_chain& chain, int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes, cudaStream_t s)
		{
			const char * what = BWD ? "bn_train_resident_kernel (backward)" : "bn_train_resident_kernel (forward)";
			size_t smem = 0;
			#define NNF_RES_CASE(A0, A1) \
				do { if (!plan_resident(p, smem, bn_train_resident_kernel<A0, A1, BWD>, n, c, hw, BWD ? 2 : 1)) return 1; \
				     return launch_resident(bn_train_resident_kernel<A0, A1, BWD>, p, smem, workspace, workspace_bytes, s, what); } while (0)
			const int k0 = chain.n > 0 ? chain.a[0].kind : NNF_ACT_NONE;
			const int k1 = chain.n > 1 ? chain.a[1].kind : NNF_ACT_NONE;
			if (chain.n == 0)
				NNF_RES_CASE(NNF_ACT_NONE, 0);
			if (chain.n == 2 && k0 == NNF_ACT_PRELU && k1 == NNF_ACT_ELU)
				NNF_RES_CASE(NNF_ACT_PRELU, NNF_ACT_ELU);
			if (chain.n == 1 && k0 == NNF_ACT_RELU)
				NNF_RES_CASE(NNF_ACT_RELU, 0);
			NNF_RES_CASE(-1, 0);
			#undef NNF_RES_CASE
		}
	}

	// Return NNF_OK after enqueueing, a negative status on an error, or 1 when the shape does not suit this kernel.
	int resident_forward_launch(cudaStream_t stream, float * y, float * saved, float * sums, const float * x, const float * gamma, const float * beta,
		float eps, const act_chain& chain, int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes)
	{
		if (!aligned16(x) || !aligned16(y))
			return 1;
		resident_params p = {};
		p.x = x; p.out = y; p.gamma = gamma; p.beta = beta; p.saved = saved; p.sums = sums;
		p.chain = chain;
		p.eps = eps;
		return resident_impl<false>(p, chain, n, c, hw, workspace, workspace_bytes, stream);
	}

	int resident_backward_launch(cudaStream_t stream, float * dx, float * bsums, const float * dy, const float * x,
		const float * gamma, const float * beta, const float * saved, const act_chain& chain,
		float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
		const float * mean, const float * invsigma, float entry_count,
		int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes)
	{
		if (!aligned16(x) || !aligned16(dy) || !aligned16(dx))
			return 1;
		resident_params p = {};
		p.x = x; p.dy = dy; p.out = dx; p.gamma = gamma; p.beta = beta; p.saved = const_cast<float *>(saved); p.sums = bsums;
		p.grad_gamma = grad_gamma; p.grad_beta = grad_beta; p.grad_mean = grad_mean; p.grad_invsigma = grad_invsigma; p.grad_slope = grad_slope;
		p.mean = mean; p.invsigma = invsigma; p.entry_count = entry_count;
		p.chain = chain;
		return resident_impl<true>(p, chain, n, c, hw, workspace, workspace_bytes, stream);
	}
}
