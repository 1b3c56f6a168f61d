// Single-launch training batch norm (+ activation chain) whose second read of x (and dy) is served
// by the L2 cache: HBM sees x (and dy) once and the result once - 8 bytes/element forward, 12
// backward - although the work is still "statistics, then normalise".
//
// One launch holds two kinds of work items, each run by one CTA of 256 threads:
//   S(channel, slice)  statistics: partial per-channel sums over a slice of the entries, written to
//                      the workspace; the item then counts itself done for its channel
//   A(channel, slice)  apply: waits until every S item of its channel is done, adds their partial sums
//                      in slice order (double, deterministic), and normalises its slice
// The items are ordered in chunks of channels: S(chunk 0), S(chunk 1), A(chunk 0), S(chunk 2),
// A(chunk 1), ... so that the A items of a chunk run while the next chunk's statistics are being
// read: the lines of x that the S items pulled in a few microseconds earlier are still in the 126 MB
// L2 (a chunk is a few tens of MB), and HBM carries a steady mix of reads and writes instead of a
// read-only kernel followed by a read-write one.
//
// A CTA does not use its block index: it draws a ticket from a global counter, and tickets are
// handed out in the order in which CTAs start running. Every S item of a channel has a smaller
// ticket than any A item of that channel, so whenever an A item waits, the items it waits for are
// already running or finished - no assumption about the order in which the hardware dispatches
// blocks, and no co-residency requirement. The wait is bounded all the same; when it runs out the
// CTA raises the library's error word (code 4) and carries on with what it has.
//
// The counters (one per channel, and the ticket) live in the caller's workspace and are cleared by
// a memset on the same stream before the launch.
//
// Batch-sharded form (one process per GPU, the same launch on every GPU): the S item that finishes a
// channel last folds this rank's partial sums and stores them, as two self-validating 8-byte words
// (32 bits of a float + the exchange's sequence number), into the mailbox of EVERY rank - plain
// peer stores over NVLink; an A item polls its OWN mailbox until the words of all ranks for its
// channel carry the sequence number, and adds them in rank order (fp32, as the other exchange forms
// do). So the exchange is per channel and overlaps the rest of the launch: no collective call, no
// kernel boundary. An S item never waits, so a rank's statistics always get published and the A
// items of every rank make progress whatever the skew between the GPUs; the wait is bounded (about a
// second; code 2), and once the error word is set the remaining waits end at once.
#include "nnf_common.cuh"

#include <stdlib.h>

namespace nnf
{
	int * device_error_word();

	namespace
	{
#ifndef NNF_CHAIN_LOADS_FWD
#define NNF_CHAIN_LOADS_FWD 4
#endif
#ifndef NNF_CHAIN_LOADS_BWD
#define NNF_CHAIN_LOADS_BWD 2
#endif
#ifndef NNF_CHAIN_MIN_CTAS
#define NNF_CHAIN_MIN_CTAS 5
#endif
		constexpr int kChainThreads = 256;
		constexpr int kChainMaxSplit = 64;     // S items per channel (sizes the partial sums)
		constexpr uint32_t kChainPollLimit = 1u << 22; // rounds of an A item's wait (about half a microsecond each)

		struct chain_params
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
			uint32_t units;              // what the items are numbered by: channels, or channel groups (grouped kernel)
			uint32_t group, groups;      // grouped kernel: channels per group, number of groups
			fastdiv d_hw;
			uint32_t split_s, entries_s; // S items per channel, entries per S item
			uint32_t split_a, entries_a; // the same for A items
			uint32_t chunk;              // channels per chunk
			uint32_t nchunks, lag;       // the A items of chunk k follow the S items of chunk k + lag
			uint32_t total_items;
			fastdiv d_vpp, d_split_s, d_split_a;
			double count;                // elements per channel
			float eps;
			// batch-sharded runs: mail[r] = mailbox of rank r (peer memory), mail[rank] this GPU's own;
			// words [2 parities][kMaxRanks source ranks][c][2]
			unsigned long long * mail[kMaxRanks];
			int rank, world;
			uint32_t seq;
			double count_total;          // elements per channel over all ranks
			double * partial;            // [c][split_s][3]
			uint32_t * done;             // [c] finished S items per channel; zero at kernel start
			uint32_t * ticket;           // zero at kernel start
			int * error;
		};

		__device__ __forceinline__ uint32_t ld_acquire(const uint32_t * p)
		{
			uint32_t v;
			asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
			return v;
		}

		__device__ __forceinline__ void st_sys_u64(unsigned long long * p, unsigned long long v)
		{
			asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
		}

		__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long * p)
		{
			unsigned long long v;
			asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
			return v;
		}

		__device__ __forceinline__ unsigned long long chain_timer_ns()
		{
			unsigned long long t;
			asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
			return t;
		}

		constexpr unsigned long long kChainPeerWaitNs = 1000000000ull; // an A item waits this long for the other ranks

		__device__ __forceinline__ size_t mail_index(const chain_params& p, uint32_t source_rank, uint32_t ch)
		{
			return ((size_t(p.seq & 1u) * kMaxRanks + source_rank) * p.c + ch) * 2;
		}

		__device__ __forceinline__ double chain_warp_sum(double v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			return v;
		}

		// Block-wide sum of K doubles; result valid in thread 0.
		template <int K>
		__device__ __forceinline__ void chain_block_sum(double (&v)[K], double * s_red)
		{
			const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
			#pragma unroll
			for (int k = 0; k < K; ++k)
				v[k] = chain_warp_sum(v[k]);
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
					for (int i = 0; i < kChainThreads / 32; ++i)
						t += s_red[i * K + k];
					v[k] = t;
				}
			}
		}

		// ticket -> (is_apply, channel, slice)
		__device__ __forceinline__ void decode_ticket(const chain_params& p, uint32_t t, uint32_t& apply, uint32_t& ch, uint32_t& sp)
		{
			uint32_t start = 0;
			for (uint32_t k = 0; k < p.nchunks + p.lag; ++k)
			{
				if (k < p.nchunks)
				{
					const uint32_t c0 = k * p.chunk;
					const uint32_t cc = min(p.chunk, p.units - c0);
					const uint32_t items = cc * p.split_s;
					if (t - start < items)
					{
						const uint32_t i = t - start;
						const uint32_t lc = p.d_split_s.div(i);
						apply = 0;
						ch = c0 + lc;
						sp = i - lc * p.split_s;
						return;
					}
					start += items;
				}
				if (k >= p.lag)
				{
					const uint32_t c0 = (k - p.lag) * p.chunk;
					const uint32_t cc = min(p.chunk, p.units - c0);
					const uint32_t items = cc * p.split_a;
					if (t - start < items)
					{
						const uint32_t i = t - start;
						const uint32_t lc = p.d_split_a.div(i);
						apply = 1;
						ch = c0 + lc;
						sp = i - lc * p.split_a;
						return;
					}
					start += items;
				}
			}
			apply = 2; // past the end: nothing to do
			ch = sp = 0;
		}

		template <int A0, int A1, bool BWD, bool PEER>
		__global__ void __launch_bounds__(kChainThreads, NNF_CHAIN_MIN_CTAS) bn_train_chain_kernel(const chain_params p)
		{
			constexpr int K = BWD ? 3 : 2;
			constexpr int kLoadsS = BWD ? NNF_CHAIN_LOADS_BWD : NNF_CHAIN_LOADS_FWD; // independent 128-bit loads in flight per thread and tensor
			constexpr int kLoadsA = kLoadsS;
			__shared__ double s_red[(kChainThreads / 32) * K];
			__shared__ uint32_t s_item[4];
			__shared__ float s_tot[4];

			if (threadIdx.x == 0)
			{
				const uint32_t t = atomicAdd(p.ticket, 1u);
				uint32_t apply, ch, sp;
				decode_ticket(p, t, apply, ch, sp);
				s_item[0] = apply;
				s_item[1] = ch;
				s_item[2] = sp;
			}
			__syncthreads();
			// the backward launch walks the channels downwards: whatever ran before it (the forward launch walks
			// upwards) left the highest channels of x in L2
			const uint32_t apply = s_item[0], ch = BWD ? p.c - 1 - s_item[1] : s_item[1], sp = s_item[2];
			if (apply > 1)
				return;
			const uint32_t per_plane = p.hw >> 2;
			const size_t entry_stride = size_t(p.c) * p.hw;

			if (!apply)
			{
				// ---- S item --------------------------------------------------------------------------
				const uint32_t e0 = sp * p.entries_s;
				const uint32_t e1 = min(e0 + p.entries_s, p.n);
				const uint32_t total = e1 > e0 ? (e1 - e0) * per_plane : 0;
				const size_t off0 = (size_t(e0) * p.c + ch) * p.hw;
				double acc[K];
				if (!BWD)
				{
					float s = 0.0F, q = 0.0F;
					for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kChainThreads * kLoadsS)
					{
						float4 a[kLoadsS];
						#pragma unroll
						for (int u = 0; u < kLoadsS; ++u)
						{
							const uint32_t i = i0 + u * kChainThreads;
							a[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
							if (i < total)
							{
								const uint32_t lp = p.d_vpp.div(i);
								a[u] = __ldg(reinterpret_cast<const float4 *>(p.x + off0 + lp * entry_stride) + (i - lp * per_plane)); // default policy: stays in L2
							}
						}
						#pragma unroll
						for (int u = 0; u < kLoadsS; ++u)
						{
							s += (a[u].x + a[u].y) + (a[u].z + a[u].w);
							q = fmaf(a[u].x, a[u].x, fmaf(a[u].y, a[u].y, fmaf(a[u].z, a[u].z, fmaf(a[u].w, a[u].w, q))));
						}
					}
					acc[0] = double(s);
					acc[1] = double(q);
				}
				else
				{
					const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
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
						sg = fmaf(du, xhat, sg);
						ss += term;
					};
					for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kChainThreads * kLoadsS)
					{
						float4 a[kLoadsS], d[kLoadsS];
						#pragma unroll
						for (int u = 0; u < kLoadsS; ++u)
						{
							const uint32_t i = i0 + u * kChainThreads;
							if (i < total)
							{
								const uint32_t lp = p.d_vpp.div(i);
								const size_t off = off0 + lp * entry_stride;
								a[u] = __ldg(reinterpret_cast<const float4 *>(p.x + off) + (i - lp * per_plane));
								d[u] = __ldg(reinterpret_cast<const float4 *>(p.dy + off) + (i - lp * per_plane));
							}
						}
						#pragma unroll
						for (int u = 0; u < kLoadsS; ++u)
							if (i0 + u * kChainThreads < total)
							{
								element(a[u].x, d[u].x); element(a[u].y, d[u].y); element(a[u].z, d[u].z); element(a[u].w, d[u].w);
							}
					}
					acc[0] = double(sb);
					acc[1] = double(sg);
					acc[2] = double(ss);
				}
				chain_block_sum<K>(acc, s_red);
				if (threadIdx.x == 0)
				{
					double * out = p.partial + (size_t(ch) * p.split_s + sp) * 3;
					#pragma unroll
					for (int k = 0; k < K; ++k)
						out[k] = acc[k];
					__threadfence(); // the partial sums are visible before the count
					const uint32_t before = atomicAdd(p.done + ch, 1u);
					if (PEER)
					{
						__threadfence(); // and the other items' partial sums are visible to this one if it is the last
						s_item[3] = before == p.split_s - 1 ? 1u : 0u;
					}
				}
				if (!PEER)
					return;
				__syncthreads();
				if (s_item[3] == 0 || threadIdx.x >= 32)
					return;
				// last S item of this channel on this rank: fold the partial sums (slice order, as the A items of
				// a single-GPU launch do), write the local per-channel outputs, publish the message to every rank
				double tot[K];
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					double t = 0.0;
					for (uint32_t q = threadIdx.x; q < p.split_s; q += 32)
						t += __ldcg(p.partial + (size_t(ch) * p.split_s + q) * 3 + k);
					tot[k] = chain_warp_sum(t);
				}
				const float m0 = float(tot[0]), m1 = float(tot[1]);
				if (threadIdx.x == 0)
				{
					if (!BWD)
					{
						if (p.sums)
						{
							p.sums[ch] = m0;
							p.sums[p.c + ch] = m1;
						}
					}
					else
					{
						const float fs = float(tot[2]);
						if (p.sums)
						{
							p.sums[ch] = m0;
							p.sums[p.c + ch] = m1;
							p.sums[2 * p.c + ch] = fs;
						}
						// per-channel gradients accumulate the LOCAL sums (batch_norm_layer_updater_cuda.cu:138-139, 167-182)
						if (p.grad_beta) p.grad_beta[ch] += m0;
						if (p.grad_gamma) p.grad_gamma[ch] += m1;
						if (p.grad_slope) p.grad_slope[ch] += fs;
					}
				}
				if (threadIdx.x < uint32_t(p.world) * 2)
				{
					__threadfence(); // everything this rank's S items wrote for the channel comes before the word
					const uint32_t r = threadIdx.x >> 1, k = threadIdx.x & 1;
					const unsigned long long word = (static_cast<unsigned long long>(p.seq) << 32) | __float_as_uint(k ? m1 : m0);
					st_sys_u64(p.mail[r] + mail_index(p, p.rank, ch) + k, word);
				}
				return;
			}

			// ---- A item ------------------------------------------------------------------------------
			const uint32_t e0 = sp * p.entries_a;
			const uint32_t e1 = min(e0 + p.entries_a, p.n);
			const uint32_t total = e1 > e0 ? (e1 - e0) * per_plane : 0;
			const size_t off0 = (size_t(e0) * p.c + ch) * p.hw;
			// position of float4 number i of this item, in floats relative to off0 (fits 32 bits: checked by the plan)
			const uint32_t entry_stride32 = p.c * p.hw;
			auto rel_of = [&](uint32_t i) -> uint32_t
			{
				const uint32_t lp = p.d_vpp.div(i);
				return lp * entry_stride32 + (i - lp * per_plane) * 4;
			};
			uint32_t rel[kLoadsA];
			// the first batch of loads does not depend on the statistics: it is issued before the wait, so
			// that the CTA has bytes in flight while it polls and folds the partial sums
			float4 a[kLoadsA];
			float4 d[BWD ? kLoadsA : 1];
			auto load_batch = [&](uint32_t i0)
			{
				#pragma unroll
				for (int u = 0; u < kLoadsA; ++u)
				{
					const uint32_t i = i0 + u * kChainThreads;
					if (i < total)
					{
						rel[u] = rel_of(i);
						a[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + off0 + rel[u]));
						if (BWD)
							d[u] = ld_stream(reinterpret_cast<const float4 *>(p.dy + off0 + rel[u]));
					}
				}
			};
			load_batch(threadIdx.x);
			if (PEER && threadIdx.x < 32)
			{
				// wait (bounded) until the words of every rank for this channel carry this exchange's number,
				// then add the messages in rank order
				const unsigned long long * mine = p.mail[p.rank];
				unsigned long long w0 = 0, w1 = 0;
				bool ok = threadIdx.x >= uint32_t(p.world);
				const unsigned long long t0 = chain_timer_ns();
				for (uint32_t round = 0; ; ++round)
				{
					if (!ok)
					{
						w0 = ld_sys_u64(mine + mail_index(p, threadIdx.x, ch));
						w1 = ld_sys_u64(mine + mail_index(p, threadIdx.x, ch) + 1);
						ok = uint32_t(w0 >> 32) == p.seq && uint32_t(w1 >> 32) == p.seq;
					}
					if (__all_sync(0xffffffffu, ok))
						break;
					bool give_up = false;
					if ((round & 15) == 15 && threadIdx.x == 0)
						give_up = (p.error && *reinterpret_cast<volatile int *>(p.error) != 0) || chain_timer_ns() - t0 > kChainPeerWaitNs;
					if (__any_sync(0xffffffffu, give_up))
					{
						if (threadIdx.x == 0 && p.error)
							*p.error = 2;
						break;
					}
					__nanosleep(200);
				}
				__threadfence(); // what the publishing items wrote before their words is visible from here on
				float f0 = 0.0F, f1 = 0.0F;
				for (int r = 0; r < p.world; ++r)
				{
					f0 += __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, w0, r)));
					f1 += __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, w1, r)));
				}
				if (threadIdx.x == 0)
				{
					if (!BWD)
					{
						const double m = double(f0) / p.count_total;
						double var = double(f1) / p.count_total - m * m;
						var = var < 0.0 ? 0.0 : var;
						const float fmean = float(m);
						const float finv = float(1.0 / sqrt(var + double(p.eps)));
						s_tot[0] = fmean;
						s_tot[1] = finv;
						if (sp == 0)
						{
							p.saved[ch] = fmean;
							p.saved[p.c + ch] = finv;
						}
					}
					else
					{
						s_tot[0] = float(double(f0) / p.count_total);
						s_tot[1] = float(double(f1) / p.count_total);
						if (sp == 0)
						{
							const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
							if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (mean - p.mean[ch]);
							if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (invstd - p.invsigma[ch]);
						}
					}
				}
			}
			if (!PEER && threadIdx.x < 32)
			{
				// wait (bounded) until every S item of this channel is done, then add their partial sums in
				// slice order: lane l takes slices l and l + 32, then a fixed shuffle tree
				bool ready = false;
				if (threadIdx.x == 0)
				{
					for (uint32_t round = 0; round < kChainPollLimit; ++round)
					{
						if (ld_acquire(p.done + ch) >= p.split_s)
						{
							ready = true;
							break;
						}
						__nanosleep(200);
					}
					if (!ready && p.error)
						*p.error = 4;
				}
				__syncwarp();
				double tot[K];
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					double t = 0.0;
					for (uint32_t q = threadIdx.x; q < p.split_s; q += 32)
						t += __ldcg(p.partial + (size_t(ch) * p.split_s + q) * 3 + k);
					tot[k] = chain_warp_sum(t);
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
						const float fb = float(tot[0]), fg = float(tot[1]), fs = float(tot[2]);
						// the same float-rounded sums the two-kernel form passes between its kernels
						s_tot[0] = float(double(fb) / p.count);
						s_tot[1] = float(double(fg) / p.count);
						if (sp == 0)
						{
							const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
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
			if (total == 0)
				return;
			const float slope = chain_slope(p.chain, ch);
			if (!BWD)
			{
				const float mean = s_tot[0], invstd = s_tot[1];
				const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
				const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
				for (uint32_t i0 = threadIdx.x; ; )
				{
					#pragma unroll
					for (int u = 0; u < kLoadsA; ++u)
					{
						const uint32_t i = i0 + u * kChainThreads;
						if (i < total)
						{
							float4 o;
							o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].x, mult), add), slope);
							o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].y, mult), add), slope);
							o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].z, mult), add), slope);
							o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].w, mult), add), slope);
							st_stream(reinterpret_cast<float4 *>(p.out + off0 + rel[u]), o);
						}
					}
					i0 += kChainThreads * kLoadsA;
					if (i0 >= total)
						break;
					load_batch(i0);
				}
			}
			else
			{
				const float c2 = s_tot[0], c3 = s_tot[1];
				const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
				const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
				const float add = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
				auto element = [&](float x, float dy) -> float
				{
					const float u = __fadd_rn(__fmul_rn(x, mult), add);
					float term;
					const float du = chain_backward<A0, A1>(p.chain, u, dy, slope, term);
					const float xhat = __fmul_rn(__fsub_rn(x, mean), invstd);
					return mult * ((du - c2) - xhat * c3);
				};
				for (uint32_t i0 = threadIdx.x; ; )
				{
					#pragma unroll
					for (int u = 0; u < kLoadsA; ++u)
					{
						const uint32_t i = i0 + u * kChainThreads;
						if (i < total)
							st_stream(reinterpret_cast<float4 *>(p.out + off0 + rel[u]),
								make_float4(element(a[u].x, d[u].x), element(a[u].y, d[u].y), element(a[u].z, d[u].z), element(a[u].w, d[u].w)));
					}
					i0 += kChainThreads * kLoadsA;
					if (i0 >= total)
						break;
					load_batch(i0);
				}
			}
		}

		// ---- the same single launch for planes that are not whole float4s (7x7, 13x13) ----------------------------
		// Items are numbered by channel GROUP: 4 / gcd(H*W, 4) adjacent channels of one entry form an aligned run of
		// whole vectors, a group is as many of those as fill the CTA's 256 vector lanes (20 channels for 7x7). A thread
		// owns one vector position of the group's run in every entry of its item, so the channels of its four
		// elements and their constants are loop invariants; an S item sums per position and folds the positions per
		// channel through shared memory, an A item folds the S items' partial sums of all the group's channels.
		constexpr int kChainGroupRun = 1024;       // floats of a group's run in one entry (one vector per thread)
		constexpr int kChainGroupChannels = 256;

		template <int A0, int A1, bool BWD, bool PEER>
		__global__ void __launch_bounds__(kChainThreads, 4) bn_train_chain_grouped_kernel(const chain_params p)
		{
			constexpr int K = BWD ? 3 : 2;
			constexpr int U = BWD ? 2 : 4;              // entries in flight per thread and tensor
			constexpr int NC = BWD ? 6 : 2;             // per-channel constants an A item derives
			constexpr uint32_t kLanes = 8;              // lanes that share a channel when sums are folded
			__shared__ float s_pos[K][kChainGroupRun];
			__shared__ float s_const[NC][kChainGroupChannels];
			__shared__ uint32_t s_item[4];

			if (threadIdx.x == 0)
			{
				const uint32_t t = atomicAdd(p.ticket, 1u);
				uint32_t apply, unit, sp;
				decode_ticket(p, t, apply, unit, sp);
				s_item[0] = apply;
				s_item[1] = unit;
				s_item[2] = sp;
				s_item[3] = 1;
			}
			__syncthreads();
			const uint32_t apply = s_item[0], grp = BWD ? p.groups - 1 - s_item[1] : s_item[1], sp = s_item[2];
			if (apply > 1)
				return;
			const uint32_t ch0 = grp * p.group;
			const uint32_t channels = min(p.group, p.c - ch0);
			const uint32_t run = channels * p.hw;
			const uint32_t v = threadIdx.x;
			const bool active = v < (run >> 2);
			const size_t stride4 = (size_t(p.c) * p.hw) >> 2;
			const uint32_t lane = threadIdx.x % kLanes;
			// channel (within the group) of each of this thread's four elements
			uint32_t local[4];
			#pragma unroll
			for (int j = 0; j < 4; ++j)
				local[j] = p.d_hw.div(min(v * 4 + j, run - 1));

			if (!apply)
			{
				// ---- S item --------------------------------------------------------------------------
				const uint32_t e0 = sp * p.entries_s;
				const uint32_t e1 = min(e0 + p.entries_s, p.n);
				const size_t base4 = (((size_t(e0) * p.c + ch0) * p.hw) >> 2) + v;
				float acc[K][4];
				#pragma unroll
				for (int k = 0; k < K; ++k)
					#pragma unroll
					for (int j = 0; j < 4; ++j)
						acc[k][j] = 0.0F;
				if constexpr (!BWD)
				{
					const float4 * bx = reinterpret_cast<const float4 *>(p.x) + base4;
					for (uint32_t e = e0; e < e1; e += U)
					{
						float4 a[U];
						#pragma unroll
						for (int u = 0; u < U; ++u)
						{
							a[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
							if (active && e + u < e1)
								a[u] = __ldg(bx + size_t(e + u - e0) * stride4); // default policy: stays in L2
						}
						#pragma unroll
						for (int u = 0; u < U; ++u)
						{
							acc[0][0] += a[u].x; acc[0][1] += a[u].y; acc[0][2] += a[u].z; acc[0][3] += a[u].w;
							acc[1][0] = fmaf(a[u].x, a[u].x, acc[1][0]); acc[1][1] = fmaf(a[u].y, a[u].y, acc[1][1]);
							acc[1][2] = fmaf(a[u].z, a[u].z, acc[1][2]); acc[1][3] = fmaf(a[u].w, a[u].w, acc[1][3]);
						}
					}
				}
				else
				{
					float mean[4], invstd[4], mult[4], add[4], slope[4];
					#pragma unroll
					for (int j = 0; j < 4; ++j)
					{
						const uint32_t ch = ch0 + local[j];
						mean[j] = __ldg(p.saved + ch);
						invstd[j] = __ldg(p.saved + p.c + ch);
						mult[j] = __fmul_rn(__ldg(p.gamma + ch), invstd[j]);
						add[j] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult[j], mean[j]));
						slope[j] = chain_slope(p.chain, ch);
					}
					const float4 * bx = reinterpret_cast<const float4 *>(p.x) + base4;
					const float4 * bd = reinterpret_cast<const float4 *>(p.dy) + base4;
					for (uint32_t e = e0; e < e1; e += U)
					{
						float4 a[U], d[U];
						#pragma unroll
						for (int u = 0; u < U; ++u)
						{
							a[u] = d[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
							if (active && e + u < e1)
							{
								a[u] = __ldg(bx + size_t(e + u - e0) * stride4);
								d[u] = __ldg(bd + size_t(e + u - e0) * stride4);
							}
						}
						#pragma unroll
						for (int u = 0; u < U; ++u)
							if (e + u < e1)
							{
								const float xs[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
								const float ds[4] = {d[u].x, d[u].y, d[u].z, d[u].w};
								#pragma unroll
								for (int j = 0; j < 4; ++j)
								{
									const float uu = __fadd_rn(__fmul_rn(xs[j], mult[j]), add[j]);
									float term;
									const float du = chain_backward<A0, A1>(p.chain, uu, ds[j], slope[j], term);
									const float xhat = __fmul_rn(__fsub_rn(xs[j], mean[j]), invstd[j]);
									acc[0][j] += du;
									acc[1][j] = fmaf(du, xhat, acc[1][j]);
									acc[2][j] += term;
								}
							}
					}
				}
				if (active)
				{
					#pragma unroll
					for (int k = 0; k < K; ++k)
						#pragma unroll
						for (int j = 0; j < 4; ++j)
							s_pos[k][v * 4 + j] = acc[k][j];
				}
				__syncthreads();
				// positions -> channels: eight lanes per channel, every eighth position each, then a butterfly
				for (uint32_t first = 0; first < channels; first += kChainThreads / kLanes)
				{
					const uint32_t lc = first + threadIdx.x / kLanes;
					double t[K];
					#pragma unroll
					for (int k = 0; k < K; ++k)
						t[k] = 0.0;
					if (lc < channels)
						for (uint32_t i = lane; i < p.hw; i += kLanes)
						{
							#pragma unroll
							for (int k = 0; k < K; ++k)
								t[k] += double(s_pos[k][lc * p.hw + i]);
						}
					#pragma unroll
					for (int k = 0; k < K; ++k)
					{
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 4);
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 2);
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 1);
					}
					if (lc < channels && lane == 0)
					{
						double * out = p.partial + (size_t(ch0 + lc) * p.split_s + sp) * 3;
						#pragma unroll
						for (int k = 0; k < K; ++k)
							out[k] = t[k];
						__threadfence(); // the partial sums are visible before the count
					}
				}
				__syncthreads();
				if (threadIdx.x == 0)
				{
					__threadfence(); // every partial sum of this item, whichever thread wrote it, comes before the count
					const uint32_t before = atomicAdd(p.done + grp, 1u);
					if (PEER)
					{
						__threadfence(); // and the other items' partial sums are visible to this one if it is the last
						s_item[3] = before == p.split_s - 1 ? 1u : 0u;
					}
				}
				if (!PEER)
					return;
				__syncthreads();
				if (s_item[3] == 0)
					return;
				// last S item of this group on this rank: fold the partial sums of every channel of the group (slice
				// order, eight lanes per channel), write the local per-channel outputs, publish the messages to every rank
				for (uint32_t first = 0; first < channels; first += kChainThreads / kLanes)
				{
					const uint32_t lc = first + threadIdx.x / kLanes;
					const uint32_t ch = ch0 + lc;
					double t[K];
					#pragma unroll
					for (int k = 0; k < K; ++k)
						t[k] = 0.0;
					if (lc < channels)
						for (uint32_t q = lane; q < p.split_s; q += kLanes)
						{
							#pragma unroll
							for (int k = 0; k < K; ++k)
								t[k] += __ldcg(p.partial + (size_t(ch) * p.split_s + q) * 3 + k);
						}
					#pragma unroll
					for (int k = 0; k < K; ++k)
					{
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 4);
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 2);
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 1);
					}
					if (lc < channels)
					{
						const float m0 = float(t[0]), m1 = float(t[1]);
						if (lane == 0)
						{
							if (p.sums)
							{
								p.sums[ch] = m0;
								p.sums[p.c + ch] = m1;
								if (BWD)
									p.sums[2 * p.c + ch] = float(t[K - 1]);
							}
							if (BWD)
							{
								// per-channel gradients accumulate the LOCAL sums (batch_norm_layer_updater_cuda.cu:138-139, 167-182)
								if (p.grad_beta) p.grad_beta[ch] += m0;
								if (p.grad_gamma) p.grad_gamma[ch] += m1;
								if (p.grad_slope) p.grad_slope[ch] += float(t[K - 1]);
							}
						}
						// lane r of the channel's eight sends both words to rank r
						if (lane < uint32_t(p.world))
						{
							__threadfence(); // everything this rank's S items wrote for the channel comes before the words
							st_sys_u64(p.mail[lane] + mail_index(p, p.rank, ch), (static_cast<unsigned long long>(p.seq) << 32) | __float_as_uint(m0));
							st_sys_u64(p.mail[lane] + mail_index(p, p.rank, ch) + 1, (static_cast<unsigned long long>(p.seq) << 32) | __float_as_uint(m1));
						}
					}
				}
				return;
			}

			// ---- A item ------------------------------------------------------------------------------
			const uint32_t e0 = sp * p.entries_a;
			const uint32_t e1 = min(e0 + p.entries_a, p.n);
			const size_t base4 = (((size_t(e0) * p.c + ch0) * p.hw) >> 2) + v;
			const float4 * bx = reinterpret_cast<const float4 *>(p.x) + base4;
			const float4 * bd = reinterpret_cast<const float4 *>(BWD ? p.dy : p.x) + base4;
			float4 * bo = reinterpret_cast<float4 *>(p.out) + base4;
			float4 a[U];
			float4 d[BWD ? U : 1];
			auto load_batch = [&](uint32_t e)
			{
				#pragma unroll
				for (int u = 0; u < U; ++u)
					if (active && e + u < e1)
					{
						a[u] = ld_stream(bx + size_t(e + u - e0) * stride4);
						if (BWD)
							d[u] = ld_stream(bd + size_t(e + u - e0) * stride4);
					}
			};
			// the first loads do not depend on the statistics: they are in flight while the item waits
			load_batch(e0);
			if constexpr (PEER)
			{
				// every channel of the group: lane r of the channel's eight waits (bounded) until rank r's two words carry this
				// exchange's number, then the messages are added in rank order
				for (uint32_t first = 0; first < channels; first += kChainThreads / kLanes)
				{
					const uint32_t lc = first + threadIdx.x / kLanes;
					const uint32_t ch = ch0 + min(lc, channels - 1);
					const unsigned long long * mine = p.mail[p.rank];
					unsigned long long w0 = 0, w1 = 0;
					bool ok = lc >= channels || lane >= uint32_t(p.world);
					const unsigned long long t0 = chain_timer_ns();
					for (uint32_t round = 0; ; ++round)
					{
						if (!ok)
						{
							w0 = ld_sys_u64(mine + mail_index(p, lane, ch));
							w1 = ld_sys_u64(mine + mail_index(p, lane, ch) + 1);
							ok = uint32_t(w0 >> 32) == p.seq && uint32_t(w1 >> 32) == p.seq;
						}
						if (__all_sync(0xffffffffu, ok))
							break;
						bool give_up = false;
						if ((round & 15) == 15 && (threadIdx.x & 31) == 0)
							give_up = (p.error && *reinterpret_cast<volatile int *>(p.error) != 0) || chain_timer_ns() - t0 > kChainPeerWaitNs;
						if (__any_sync(0xffffffffu, give_up))
						{
							if ((threadIdx.x & 31) == 0 && p.error)
								*p.error = 2;
							break;
						}
						__nanosleep(200);
					}
					__threadfence(); // what the publishing items wrote before their words is visible from here on
					float f0 = 0.0F, f1 = 0.0F;
					const int lane0 = int(threadIdx.x & 31u) & ~int(kLanes - 1);   // first lane of this channel's eight
					for (int r = 0; r < p.world; ++r)
					{
						f0 += __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, w0, lane0 + r)));
						f1 += __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, w1, lane0 + r)));
					}
					if (lc < channels && lane == 0)
					{
						if constexpr (!BWD)
						{
							const double m = double(f0) / p.count_total;
							double var = double(f1) / p.count_total - m * m;
							var = var < 0.0 ? 0.0 : var;
							const float fmean = float(m);
							const float finv = float(1.0 / sqrt(var + double(p.eps)));
							const float mult = __fmul_rn(__ldg(p.gamma + ch), finv);
							s_const[0][lc] = mult;
							s_const[1][lc] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, fmean));
							if (sp == 0)
							{
								p.saved[ch] = fmean;
								p.saved[p.c + ch] = finv;
							}
						}
						else
						{
							const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
							const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
							s_const[0][lc] = mult;
							s_const[1][lc] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
							s_const[NC - 4][lc] = mean;
							s_const[NC - 3][lc] = invstd;
							s_const[NC - 2][lc] = float(double(f0) / p.count_total);
							s_const[NC - 1][lc] = float(double(f1) / p.count_total);
							if (sp == 0)
							{
								if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (mean - p.mean[ch]);
								if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (invstd - p.invsigma[ch]);
							}
						}
					}
				}
			}
			if (!PEER && threadIdx.x == 0)
			{
				bool ready = false;
				for (uint32_t round = 0; round < kChainPollLimit; ++round)
				{
					if (ld_acquire(p.done + grp) >= p.split_s)
					{
						ready = true;
						break;
					}
					__nanosleep(200);
				}
				if (!ready && p.error)
					*p.error = 4;
			}
			__syncthreads();
			// the S items' partial sums of every channel of the group, in slice order: eight lanes per channel
			for (uint32_t first = 0; !PEER && first < channels; first += kChainThreads / kLanes)
			{
				const uint32_t lc = first + threadIdx.x / kLanes;
				const uint32_t ch = ch0 + lc;
				double t[K];
				#pragma unroll
				for (int k = 0; k < K; ++k)
					t[k] = 0.0;
				if (lc < channels)
					for (uint32_t q = lane; q < p.split_s; q += kLanes)
					{
						#pragma unroll
						for (int k = 0; k < K; ++k)
							t[k] += __ldcg(p.partial + (size_t(ch) * p.split_s + q) * 3 + k);
					}
				#pragma unroll
				for (int k = 0; k < K; ++k)
				{
					t[k] += __shfl_xor_sync(0xffffffffu, t[k], 4);
					t[k] += __shfl_xor_sync(0xffffffffu, t[k], 2);
					t[k] += __shfl_xor_sync(0xffffffffu, t[k], 1);
				}
				if (lc < channels && lane == 0)
				{
					if constexpr (!BWD)
					{
						const double m = t[0] / p.count;
						double var = t[1] / p.count - m * m;
						var = var < 0.0 ? 0.0 : var;
						const float fmean = float(m);
						const float finv = float(1.0 / sqrt(var + double(p.eps)));
						const float mult = __fmul_rn(__ldg(p.gamma + ch), finv);
						s_const[0][lc] = mult;
						s_const[1][lc] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, fmean));
						if (sp == 0)
						{
							p.saved[ch] = fmean;
							p.saved[p.c + ch] = finv;
							if (p.sums)
							{
								p.sums[ch] = float(t[0]);
								p.sums[p.c + ch] = float(t[1]);
							}
						}
					}
					else
					{
						const float fb = float(t[0]), fg = float(t[1]), fs = float(t[K - 1]);
						const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
						const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
						s_const[0][lc] = mult;
						s_const[1][lc] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
						s_const[NC - 4][lc] = mean;
						s_const[NC - 3][lc] = invstd;
						// the same float-rounded sums the two-kernel form passes between its kernels
						s_const[NC - 2][lc] = float(double(fb) / p.count);
						s_const[NC - 1][lc] = float(double(fg) / p.count);
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
			if (!active || e0 >= e1)
				return;
			float mult[4], add[4], slope[4];
			#pragma unroll
			for (int j = 0; j < 4; ++j)
			{
				mult[j] = s_const[0][local[j]];
				add[j] = s_const[1][local[j]];
				slope[j] = chain_slope(p.chain, ch0 + local[j]);
			}
			if constexpr (!BWD)
			{
				for (uint32_t e = e0; ; )
				{
					#pragma unroll
					for (int u = 0; u < U; ++u)
						if (e + u < e1)
						{
							float4 o;
							o.x = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].x, mult[0]), add[0]), slope[0]);
							o.y = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].y, mult[1]), add[1]), slope[1]);
							o.z = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].z, mult[2]), add[2]), slope[2]);
							o.w = chain_forward<A0, A1>(p.chain, __fadd_rn(__fmul_rn(a[u].w, mult[3]), add[3]), slope[3]);
							st_stream(bo + size_t(e + u - e0) * stride4, o);
						}
					e += U;
					if (e >= e1)
						break;
					load_batch(e);
				}
			}
			else
			{
				float mean[4], invstd[4], c2[4], c3[4];
				#pragma unroll
				for (int j = 0; j < 4; ++j)
				{
					mean[j] = s_const[NC - 4][local[j]];
					invstd[j] = s_const[NC - 3][local[j]];
					c2[j] = s_const[NC - 2][local[j]];
					c3[j] = s_const[NC - 1][local[j]];
				}
				for (uint32_t e = e0; ; )
				{
					#pragma unroll
					for (int u = 0; u < U; ++u)
						if (e + u < e1)
						{
							const float xs[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
							const float ds[4] = {d[u].x, d[u].y, d[u].z, d[u].w};
							float rs[4];
							#pragma unroll
							for (int j = 0; j < 4; ++j)
							{
								const float uu = __fadd_rn(__fmul_rn(xs[j], mult[j]), add[j]);
								float term;
								const float du = chain_backward<A0, A1>(p.chain, uu, ds[j], slope[j], term);
								const float xhat = __fmul_rn(__fsub_rn(xs[j], mean[j]), invstd[j]);
								rs[j] = mult[j] * ((du - c2[j]) - xhat * c3[j]);
							}
							st_stream(bo + size_t(e + u - e0) * stride4, make_float4(rs[0], rs[1], rs[2], rs[3]));
						}
					e += U;
					if (e >= e1)
						break;
					load_batch(e);
				}
			}
		}

		int chain_env(const char * name, int fallback)
		{
			const char * v = getenv(name);
			return v ? atoi(v) : fallback;
		}

		// Item sizes and chunking. Defaults measured on B200 with x[256,256,28,28], PReLU+ELU (forward / backward):
		// S 48 KB, A 64 KB, 16 MB chunks, lag 1: 95 / 154 us; A 32 KB: 99 / 178 us; S 96 KB: 96 / 170 us; chunk 8 MB:
		// 122 / 216 us (apply items catch up with their statistics); lag 0: 124 / 227 us. Loads in flight per
		// thread (4 / 2 per tensor against 8 / 4) and CTAs per SM (4 to 6) change the times by a few percent only.
		// Tuning aids: NNF_CHAIN_S_KB / NNF_CHAIN_A_KB (bytes of one tensor that an
		// S / A item covers), NNF_CHAIN_CHUNK_MB (bytes of one tensor per chunk), NNF_CHAIN_LAG.
		bool plan_chain(chain_params& p, int64_t n, int64_t c, int64_t hw, int tensors)
		{
			(void)tensors;
			if (hw % 4 != 0 || n < 1 || c < 1 || n * hw >= (int64_t(1) << 31) || c > 0x7fffffff / 256)
				return false;
			const int64_t plane_bytes = hw * 4;
			const int64_t s_bytes = int64_t(chain_env("NNF_CHAIN_S_KB", 48)) * 1024;
			const int64_t a_bytes = int64_t(chain_env("NNF_CHAIN_A_KB", 64)) * 1024;
			int64_t es = s_bytes / plane_bytes, ea = a_bytes / plane_bytes;
			if (es < 1) es = 1;
			if (ea < 1) ea = 1;
			if (es > n) es = n;
			if (ea > n) ea = n;
			if (div_up(n, es) > kChainMaxSplit)
				es = div_up(n, kChainMaxSplit);
			if (div_up(n, ea) > 4096)
				ea = div_up(n, 4096);
			p.entries_s = (uint32_t)es;
			p.split_s = (uint32_t)div_up(n, es);
			if (ea * c * hw >= (int64_t(1) << 32))
				return false; // positions inside an apply item are kept in 32 bits
			p.entries_a = (uint32_t)ea;
			p.split_a = (uint32_t)div_up(n, ea);
			const double channel_bytes = double(n) * double(plane_bytes);
			int64_t chunk = (int64_t)(double(chain_env("NNF_CHAIN_CHUNK_MB", 16)) * 1024.0 * 1024.0 / channel_bytes);
			if (chunk < 1) chunk = 1;
			if (chunk < div_up(c, 64)) chunk = div_up(c, 64); // at most 64 chunks: a CTA finds its item by walking them
			if (chunk > c) chunk = c;
			p.chunk = (uint32_t)chunk;
			p.nchunks = (uint32_t)div_up(c, chunk);
			int lag = chain_env("NNF_CHAIN_LAG", 1);
			p.lag = (uint32_t)(lag < 0 ? 0 : lag);
			const int64_t items = c * (int64_t(p.split_s) + int64_t(p.split_a));
			if (items >= (int64_t(1) << 31) || p.nchunks + p.lag > 4096)
				return false;
			p.total_items = (uint32_t)items;
			p.n = (uint32_t)n; p.c = (uint32_t)c; p.hw = (uint32_t)hw;
			p.units = p.c;
			p.d_vpp = fastdiv((uint32_t)(hw / 4));
			p.d_split_s = fastdiv(p.split_s);
			p.d_split_a = fastdiv(p.split_a);
			p.count = double(n) * double(hw);
			return true;
		}

		// The grouped kernel's plan: items are channel groups. Returns false where the shape does not suit it (planes
		// of whole float4s take the kernel above; runs shorter than 16 vectors or longer than 256 the separate kernels).
		bool plan_chain_grouped(chain_params& p, int64_t n, int64_t c, int64_t hw)
		{
			if (hw % 4 == 0 || n < 1 || c < 1 || n >= (int64_t(1) << 31) || c >= (int64_t(1) << 24) || getenv("NNF_NO_GROUPED_CHAIN"))
				return false;
			const int64_t unit = (hw % 2 == 0) ? 2 : 4;
			const int64_t vpu = unit * hw / 4;
			if (c % unit != 0 || vpu > kChainThreads)
				return false;
			int64_t group = unit * (kChainThreads / vpu);
			if (group > c) group = c;
			if (group > kChainGroupChannels) group = kChainGroupChannels;
			if (group * hw / 4 < 16)
				return false;
			const int64_t groups = div_up(c, group);
			const int64_t run_bytes = group * hw * 4;
			const int64_t s_bytes = int64_t(chain_env("NNF_CHAIN_S_KB", 48)) * 1024;
			const int64_t a_bytes = int64_t(chain_env("NNF_CHAIN_A_KB", 64)) * 1024;
			int64_t es = s_bytes / run_bytes, ea = a_bytes / run_bytes;
			if (es < 1) es = 1;
			if (ea < 1) ea = 1;
			if (es > n) es = n;
			if (ea > n) ea = n;
			if (div_up(n, es) > kChainMaxSplit)
				es = div_up(n, kChainMaxSplit);
			if (div_up(n, ea) > 4096)
				ea = div_up(n, 4096);
			p.entries_s = (uint32_t)es;
			p.split_s = (uint32_t)div_up(n, es);
			p.entries_a = (uint32_t)ea;
			p.split_a = (uint32_t)div_up(n, ea);
			const double group_bytes = double(n) * double(run_bytes);
			int64_t chunk = (int64_t)(double(chain_env("NNF_CHAIN_CHUNK_MB", 16)) * 1024.0 * 1024.0 / group_bytes);
			if (chunk < 1) chunk = 1;
			if (chunk < div_up(groups, 64)) chunk = div_up(groups, 64);
			if (chunk > groups) chunk = groups;
			p.chunk = (uint32_t)chunk;
			p.nchunks = (uint32_t)div_up(groups, chunk);
			int lag = chain_env("NNF_CHAIN_LAG", 1);
			p.lag = (uint32_t)(lag < 0 ? 0 : lag);
			const int64_t items = groups * (int64_t(p.split_s) + int64_t(p.split_a));
			if (items >= (int64_t(1) << 31))
				return false;
			p.total_items = (uint32_t)items;
			p.n = (uint32_t)n; p.c = (uint32_t)c; p.hw = (uint32_t)hw;
			p.units = (uint32_t)groups;
			p.group = (uint32_t)group;
			p.groups = (uint32_t)groups;
			p.d_hw = fastdiv((uint32_t)hw);
			p.d_split_s = fastdiv(p.split_s);
			p.d_split_a = fastdiv(p.split_a);
			p.count = double(n) * double(hw);
			return true;
		}

		size_t chain_workspace_needed(const chain_params& p)
		{
			return size_t(p.c) * p.split_s * 3 * sizeof(double) + (size_t(p.c) + 1) * sizeof(uint32_t);
		}

		template <class Kernel>
		int launch_chain(Kernel kernel, chain_params& p, void * workspace, cudaStream_t s, const char * what)
		{
			p.partial = static_cast<double *>(workspace);
			p.done = reinterpret_cast<uint32_t *>(p.partial + size_t(p.c) * p.split_s * 3);
			p.ticket = p.done + p.c;
			p.error = device_error_word();
			cudaError_t e = cudaMemsetAsync(p.done, 0, (size_t(p.c) + 1) * sizeof(uint32_t), s);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s: cudaMemsetAsync: %s", what, cudaGetErrorString(e));
			kernel<<<p.total_items, kChainThreads, 0, s>>>(p);
			return check_launch(what);
		}
	}

	size_t chain_workspace_bytes(int64_t c)
	{
		return size_t(c) * kChainMaxSplit * 3 * sizeof(double) + (size_t(c) + 1) * sizeof(uint32_t);
	}

	namespace
	{
		struct chain_peer
		{
			void * const * mailboxes;
			int rank, world;
			uint32_t seq;
			double count_total;
		};

		int fill_peer(chain_params& p, const chain_peer * peer, const char * who)
		{
			p.count_total = p.count;
			if (!peer)
				return NNF_OK;
			if (peer->world < 1 || peer->world > kMaxRanks || peer->rank < 0 || peer->rank >= peer->world || !peer->mailboxes || peer->seq == 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: bad peer arguments (rank %d of %d, sequence number %u; at most %d ranks, numbers start at 1)",
					who, peer->rank, peer->world, peer->seq, kMaxRanks);
			for (int r = 0; r < peer->world; ++r)
			{
				if (!peer->mailboxes[r] || (reinterpret_cast<uintptr_t>(peer->mailboxes[r]) & 7))
					return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: mailbox of rank %d is null or not 8-byte aligned", who, r);
				p.mail[r] = static_cast<unsigned long long *>(peer->mailboxes[r]);
			}
			p.rank = peer->rank;
			p.world = peer->world;
			p.seq = peer->seq;
			p.count_total = peer->count_total;
			return NNF_OK;
		}

		template <bool PEER>
		int chain_forward_impl(cudaStream_t stream, float * y, float * saved, float * sums, const float * x, const float * gamma, const float * beta,
			float eps, const act_chain& chain, int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes, const chain_peer * peer)
		{
			chain_params p = {};
			if (!aligned16(x) || !aligned16(y))
				return 1;
			const bool grouped = plan_chain_grouped(p, n, c, hw);
			if (!grouped && !plan_chain(p, n, c, hw, 1))
				return 1;
			if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 7) || workspace_bytes < chain_workspace_needed(p))
				return 1;
			p.x = x; p.out = y; p.gamma = gamma; p.beta = beta; p.saved = saved; p.sums = sums;
			p.chain = chain;
			p.eps = eps;
			const int st = fill_peer(p, peer, "bn_train_chain_kernel (forward)");
			if (st != NNF_OK)
				return st;
			if (grouped)
			{
				const char * what = "bn_train_chain_grouped_kernel (forward)";
				switch (chain_id(chain))
				{
				case 0: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_NONE, 0, false, PEER>, p, workspace, stream, what);
				case 1: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, false, PEER>, p, workspace, stream, what);
				case 2: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_RELU, 0, false, PEER>, p, workspace, stream, what);
				default: return launch_chain(bn_train_chain_grouped_kernel<-1, 0, false, PEER>, p, workspace, stream, what);
				}
			}
			const int k0 = chain.n > 0 ? chain.a[0].kind : NNF_ACT_NONE;
			const int k1 = chain.n > 1 ? chain.a[1].kind : NNF_ACT_NONE;
			if (chain.n == 0)
				return launch_chain(bn_train_chain_kernel<NNF_ACT_NONE, 0, false, PEER>, p, workspace, stream, "bn_train_chain_kernel (forward)");
			if (k0 == NNF_ACT_PRELU && k1 == NNF_ACT_ELU && chain.n == 2)
				return launch_chain(bn_train_chain_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, false, PEER>, p, workspace, stream, "bn_train_chain_kernel (forward)");
			if (k0 == NNF_ACT_RELU && chain.n == 1)
				return launch_chain(bn_train_chain_kernel<NNF_ACT_RELU, 0, false, PEER>, p, workspace, stream, "bn_train_chain_kernel (forward)");
			return launch_chain(bn_train_chain_kernel<-1, 0, false, PEER>, p, workspace, stream, "bn_train_chain_kernel (forward)");
		}

		template <bool PEER>
		int chain_backward_impl(cudaStream_t stream, float * dx, float * bsums, const float * dy, const float * x,
			const float * gamma, const float * beta, const float * saved, const act_chain& chain,
			float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
			const float * mean, const float * invsigma, float entry_count,
			int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes, const chain_peer * peer)
		{
			chain_params p = {};
			if (!aligned16(x) || !aligned16(dy) || !aligned16(dx))
				return 1;
			const bool grouped = plan_chain_grouped(p, n, c, hw);
			if (!grouped && !plan_chain(p, n, c, hw, 2))
				return 1;
			if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 7) || workspace_bytes < chain_workspace_needed(p))
				return 1;
			p.x = x; p.dy = dy; p.out = dx; p.gamma = gamma; p.beta = beta; p.saved = const_cast<float *>(saved); p.sums = bsums;
			p.grad_gamma = grad_gamma; p.grad_beta = grad_beta; p.grad_mean = grad_mean; p.grad_invsigma = grad_invsigma; p.grad_slope = grad_slope;
			p.mean = mean; p.invsigma = invsigma; p.entry_count = entry_count;
			p.chain = chain;
			const int st = fill_peer(p, peer, "bn_train_chain_kernel (backward)");
			if (st != NNF_OK)
				return st;
			if (grouped)
			{
				const char * what = "bn_train_chain_grouped_kernel (backward)";
				switch (chain_id(chain))
				{
				case 0: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_NONE, 0, true, PEER>, p, workspace, stream, what);
				case 1: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, true, PEER>, p, workspace, stream, what);
				case 2: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_RELU, 0, true, PEER>, p, workspace, stream, what);
				default: return launch_chain(bn_train_chain_grouped_kernel<-1, 0, true, PEER>, p, workspace, stream, what);
				}
			}
			switch (chain_id(chain))
			{
			case 0: return launch_chain(bn_train_chain_kernel<NNF_ACT_NONE, 0, true, PEER>, p, workspace, stream, "bn_train_chain_kernel (backward)");
			case 1: return launch_chain(bn_train_chain_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, true, PEER>, p, workspace, stream, "bn_train_chain_kernel (backward)");
			case 2: return launch_chain(bn_train_chain_kernel<NNF_ACT_RELU, 0, true, PEER>, p, workspace, stream, "bn_train_chain_kernel (backward)");
			default: return launch_chain(bn_train_chain_kernel<-1, 0, true, PEER>, p, workspace, stream, "bn_train_chain_kernel (backward)");
			}
		}
	}

	// Returns NNF_OK after enqueueing, a negative status on an error, or 1 when the shape does not suit
	// this kernel (the caller then uses another form).
	int chain_forward_launch(cudaStream_t stream, float * y, float * saved, float * sums, const float * x, const float * gamma, const float * beta,
		float eps, const act_chain& chain, int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes)
	{
		return chain_forward_impl<false>(stream, y, saved, sums, x, gamma, beta, eps, chain, n, c, hw, workspace, workspace_bytes, nullptr);
	}

	int chain_backward_launch(cudaStream_t stream, float * dx, float * bsums, const float * dy, const float * x,
		const float * gamma, const float * beta, const float * saved, const act_chain& chain,
		float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
		const float * mean, const float * invsigma, float entry_count,
		int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes)
	{
		return chain_backward_impl<false>(stream, dx, bsums, dy, x, gamma, beta, saved, chain, grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope,
			mean, invsigma, entry_count, n, c, hw, workspace, workspace_bytes, nullptr);
	}
}

using namespace nnf;

extern "C" int nnf_bn_train_sharded_supported(int64_t n, int64_t c, int64_t hw)
{
	chain_params p = {};
	return (plan_chain_grouped(p, n, c, hw) || plan_chain(p, n, c, hw, 1)) ? 1 : 0;
}

extern "C" size_t nnf_bn_train_mailbox_bytes(int64_t c)
{
	return c > 0 ? size_t(2) * kMaxRanks * size_t(c) * 2 * sizeof(unsigned long long) : 0;
}

extern "C" int nnf_bn_train_fwd_sharded(nnf_stream_t stream, float * y, float * saved, float * sums, const float * x,
	const float * gamma, const float * beta, float eps, const nnf_act * acts, int n_acts,
	int64_t n, int64_t c, int64_t hw, double count_total, void * workspace, size_t workspace_bytes,
	void * const * mailboxes, int rank, int world, uint32_t seq)
{
	if (n <= 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_fwd_sharded: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (!y || !x || !gamma || !beta || !saved)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_fwd_sharded: null pointer");
	act_chain chain;
	int st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	const chain_peer peer = {mailboxes, rank, world, seq, count_total};
	st = chain_forward_impl<true>((cudaStream_t)stream, y, saved, sums, x, gamma, beta, eps, chain, n, c, hw, workspace, workspace_bytes, &peer);
	if (st == 1)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_fwd_sharded: needs a shape for which nnf_bn_train_sharded_supported() answers 1, 16-byte aligned tensors and a workspace of nnf_bn_train_workspace_bytes()");
	return st;
}

extern "C" int nnf_bn_train_bwd_sharded(nnf_stream_t stream, float * dx, float * bsums, const float * dy, const float * x,
	const float * gamma, const float * beta, const float * saved, const nnf_act * acts, int n_acts,
	float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
	const float * mean, const float * invsigma, float entry_count,
	int64_t n, int64_t c, int64_t hw, double count_total, void * workspace, size_t workspace_bytes,
	void * const * mailboxes, int rank, int world, uint32_t seq)
{
	if (n <= 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_sharded: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (!dx || !dy || !x || !gamma || !beta || !saved || !bsums)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_sharded: null pointer");
	if ((grad_mean && !mean) || (grad_invsigma && !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_bwd_sharded: running-statistics gradients requested without the running statistics");
	act_chain chain;
	int st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	chain_fill_backward_constants(chain, acts, n_acts);
	int prelus = 0;
	for (int i = 0; i < chain.n; ++i)
		prelus += chain.a[i].kind == NNF_ACT_PRELU;
	if (prelus > 1)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_bwd_sharded: at most one PReLU per fused chain");
	const chain_peer peer = {mailboxes, rank, world, seq, count_total};
	st = chain_backward_impl<true>((cudaStream_t)stream, dx, bsums, dy, x, gamma, beta, saved, chain, grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope,
		mean, invsigma, entry_count, n, c, hw, workspace, workspace_bytes, &peer);
	if (st == 1)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_bwd_sharded: needs a shape for which nnf_bn_train_sharded_supported() answers 1, 16-byte aligned tensors and a workspace of nnf_bn_train_workspace_bytes()");
	return st;
}
