// Single-launch training batch norm (+ activation chain) whose second read of x (and dy) is served
// by the L2 cache: HBM sees x (and dy) once and the result once - 8 bytes/element forward, 12
// backward - although the work is still "statistics, then normalise".
//
// One launch holds three kinds of work items, each run by one CTA of 256 threads that draws a ticket
// from a global counter (tickets are handed out in the order in which CTAs start running, so no
// assumption is made about the order in which the hardware dispatches blocks):
//   S(channel, slice)  statistics over a slice of the entries: every warp leaves its partial sums in the
//                      workspace as 8-byte words that carry the launch's tag next to the value, so a
//                      reader can tell them from stale ones - no counter, no fence, nothing to wait for
//   F(channel)         one warp: waits (bounded) until every deposit of the channel carries the tag, adds
//                      them in a fixed order in double, derives the channel's constants (and writes the
//                      per-channel outputs), releases the channel's apply items
//   A(channel, slice)  apply: issues its first copies, then waits (bounded) for F(channel), normalises
// Ticket step k holds S(k), F(k - dist/2) and A(k - dist), interleaved, so that the apply items of a
// channel run while later channels' statistics are being read: the lines of x that the S items pulled in
// a few microseconds earlier are still in the 126 MB L2 (they are loaded with an evict-last hint, the
// second read with evict-first, the result with streaming stores), and HBM carries a steady mix of
// reads and writes. Every item with a smaller ticket than a waiting one is running or finished, so the
// waits cannot deadlock; they are bounded all the same, and on expiry the launch's own status word (in
// the workspace, cleared by the memset that precedes every launch) is raised and the launch finishes
// with what it has.
//
// Global memory reaches the threads through shared memory without occupying registers: a thread copies
// its 16-byte pieces of the next sweeps with cp.async into slots that only it reads back (no barrier),
// three sweeps ahead. A sweep is as many whole planes of the channel (consecutive entries) as fill
// the CTA's vector slots (1024 forward; 512 backward, where two tensors are staged, so that four CTAs
// fit an SM in both directions); a thread's slot offsets inside a sweep never change, so the loop has no
// index division.
//
// Batch-sharded form (one process per GPU, the same launch on every GPU): F(channel) folds this rank's
// deposits, stores the rank's two sums into the mailbox of EVERY rank as two self-validating 8-byte
// words (32 bits of a float + the exchange's sequence number; plain peer stores over NVLink), waits
// (bounded by the configured limit) until its own mailbox holds the words of all ranks, adds them in
// rank order and releases the apply items. Only the finishing warps ever look at peer memory; S items
// never wait, so a rank's statistics always get published whatever the skew between the GPUs.
//
// Planes that are not whole float4s (7x7, 13x13) take the channel-group kernel further down, whose
// items follow an older scheme (counters, chunks of channel groups, apply items that fold the sums).
#include "nnf_common.cuh"

#include <atomic>
#include <mutex>

namespace nnf
{
	int * device_error_word();

	namespace
	{
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
			float * fin;                 // [c][8] one GPU: the constants a group's last S item leaves for its A items
			uint32_t * done;             // [groups] finished S items per group, then [groups] flags "constants written"; zero at kernel start
			uint32_t * ticket;           // zero at kernel start
			int * error;                 // the launch's status word (in the workspace head; zero at kernel start)
			int * error_word;            // the library's process-wide word: raised too, never consulted
			unsigned long long wait_limit_ns;
			unsigned long long * wait_ns; // the launch report's {sum, longest} of the waits for other ranks
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

		constexpr unsigned long long kDefaultPeerWaitNs = 10000000000ull; // a launch waits this long for another rank's statistics unless told otherwise

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

		// ---- the kernel for planes of whole float4s ------------------------------------------------------------
		constexpr int kStreamSlots = 4;                 // 16-byte slots of a thread in one sweep (forward)
		constexpr int kStreamSlotsBwd = 2;              // the same, backward: two tensors are staged
		constexpr int kStreamWarps = kChainThreads / 32;
		constexpr int kStagesFwd = 3, kStagesBwd = 3;   // sweeps in flight per thread (48 KB of shared memory per CTA in both directions)
		constexpr int kCtasFwd = 4, kCtasBwd = 4;       // resident CTAs per SM the register budget is cut for

		// The head of every workspace: what a launch reports. Cleared by the memset in front of the launch.
		struct launch_report
		{
			unsigned long long wait_ns_total;   // time the waiting items spent waiting, summed
			unsigned long long wait_ns_max;     // the longest single wait
			uint32_t reserved;
			int status;                         // 0, or the code of the bounded wait that ran out (2: another rank, 4: this GPU's own items)
			uint32_t pad0[26];
			uint32_t ticket;                    // every CTA of the launch draws from it: alone on its 128-byte line
			uint32_t pad1[31];
		};
		static_assert(sizeof(launch_report) == 256, "the report is two 128-byte lines");

		struct stream_params
		{
			const float * x;
			const float * dy;        // backward only
			float * out;             // y (forward) or dx (backward)
			const float * gamma;
			const float * beta;
			float * saved;           // forward: written {mean, invstd}; backward: read
			float * sums;            // forward: {sum x, sum x^2} of this shard (may be null); backward: bsums[3C]
			float * grad_gamma, * grad_beta, * grad_mean, * grad_invsigma, * grad_slope;
			const float * mean, * invsigma;
			float entry_count;
			act_chain chain;
			uint32_t n, c, hw, vpp;
			uint32_t rows, cols, tiles;        // a sweep: `rows` whole planes of `cols` vectors, or one column tile of a wide plane
			uint32_t es, ea, ss, sa;           // entries per S / A item, items per channel
			uint32_t dist, dist_f;             // A(k - dist) and F(k - dist_f) share ticket step k with S(k)
			uint32_t total;
			fastdiv d_cols, d_per, d_both, d_rows;
			double count, count_total;         // elements per channel on this rank / over all ranks
			float eps;
			uint32_t tag;                      // this launch's tag in the deposit words
			unsigned long long * deposit;      // [c][ss][4] tagged words
			float4 * fin;                      // [c][2] per-channel constants for the A items
			uint32_t * ready;                  // [c]
			launch_report * report;
			int * error_word;                  // the library's process-wide word: raised too, never consulted
			// batch-sharded runs: mail[r] = mailbox of rank r (peer memory), mail[rank] this GPU's own;
			// words [2 parities][kMaxRanks source ranks][c][2]
			unsigned long long * mail[kMaxRanks];
			int rank, world;
			uint32_t seq;
			unsigned long long wait_limit_ns;
		};

		__device__ __forceinline__ void st_relaxed_u64(unsigned long long * p, unsigned long long v)
		{
			asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
		}

		__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long * p)
		{
			unsigned long long v;
			asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
			return v;
		}

		__device__ __forceinline__ void st_release_u32(uint32_t * p, uint32_t v)
		{
			asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
		}

		__device__ __forceinline__ void cp_async16(void * dst_smem, const char * src, uint64_t policy)
		{
			asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;"
				:: "r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src), "l"(policy) : "memory");
		}

		__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

		template <int N>
		__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

		__device__ __forceinline__ float stream_warp_sum(float v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			return v;
		}

		__device__ __forceinline__ size_t mail_index(const stream_params& p, uint32_t source_rank, uint32_t ch)
		{
			return ((size_t(p.seq & 1u) * kMaxRanks + source_rank) * p.c + ch) * 2;
		}

		// Backward through the chain from u = bn output: returns du, `term` = the PReLU slope gradient's term. PReLU
		// followed by ELU, the chain the kernel is measured on, has a shorter form: the ELU's derivative for a
		// negative input, (e^t - 1) + 1 in the layer-by-layer arithmetic, is taken as e^t itself (they differ by
		// one rounding of a number near 1, far inside the tolerance of this row).
		template <int A0, int A1>
		__device__ __forceinline__ float stream_backward(const act_chain& ch, float u, float dy, float slope, float& term)
		{
			if constexpr (A0 == NNF_ACT_PRELU && A1 == NNF_ACT_ELU)
			{
				const float k = u >= 0.0F ? 1.0F : slope;
				const float t1 = u * k;
				const float e = fast_exp(t1);
				const float g = dy * (t1 >= 0.0F ? 1.0F : e);
				term = g * fminf(u, 0.0F);
				return g * k;
			}
			else
				return chain_backward<A0, A1>(ch, u, dy, slope, term);
		}

		template <int A0, int A1, bool BWD, bool PEER>
		__global__ void __launch_bounds__(kChainThreads, BWD ? kCtasBwd : kCtasFwd) bn_train_chain_kernel(const stream_params p)
		{
			constexpr int K = BWD ? 3 : 2;
			constexpr int T = BWD ? 2 : 1;
			constexpr int L = BWD ? kStreamSlotsBwd : kStreamSlots;
			constexpr int STAGES = BWD ? kStagesBwd : kStagesFwd;
			extern __shared__ float4 ring[];   // [STAGES][T][L][kChainThreads]: a thread reads back only what it copied itself
			__shared__ uint32_t s_item[4];
			__shared__ float4 s_fin[2];
			__shared__ float s_sum[kStreamWarps][3];

			if (threadIdx.x == 0)
			{
				// step k of the ticket order holds the finishing item of channel k - dist_f, then the statistics items of
				// channel k and the apply items of channel k - dist, interleaved; items of channels outside [0, c) are empty
				const uint32_t t = atomicAdd(&p.report->ticket, 1u);
				uint32_t kind = 3, chq = 0, sp = 0;
				const uint32_t per = p.ss + p.sa + 1;
				const uint32_t step = p.d_per.div(t);
				const uint32_t i = t - step * per;
				if (i == 0)
				{
					if (step >= p.dist_f && step - p.dist_f < p.c) { kind = 2; chq = step - p.dist_f; }
				}
				else
				{
					const uint32_t j = i - 1;
					const uint32_t s0 = p.d_both.div(j * p.ss), s1 = p.d_both.div((j + 1) * p.ss);
					if (s1 > s0) { if (step < p.c) { kind = 0; chq = step; sp = s0; } }
					else if (step >= p.dist && step - p.dist < p.c) { kind = 1; chq = step - p.dist; sp = j - s0; }
				}
				s_item[0] = kind; s_item[1] = chq; s_item[2] = sp;
			}
			__syncthreads();
			// the backward launch walks the channels downwards: whatever ran before it (the forward launch walks
			// upwards) left the highest channels of x in L2
			const uint32_t kind = s_item[0], ch = BWD ? p.c - 1 - s_item[1] : s_item[1], sp = s_item[2];
			if (kind > 2)
				return;
			const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
			const uint32_t deposits = p.ss;

			if (kind == 2)
			{
				// ---- F item ------------------------------------------------------------------------------
				if (warp != 0)
					return;
				const unsigned long long * part = p.deposit + size_t(ch) * deposits * 4;
				double tot[K];
				bool ok = false;
				const unsigned long long t0 = chain_timer_ns();
				for (uint32_t round = 0; round < kChainPollLimit; ++round)
				{
					bool all = true;
					#pragma unroll
					for (int k = 0; k < K; ++k)
						tot[k] = 0.0;
					for (uint32_t e = lane; e < deposits; e += 32)
					{
						#pragma unroll
						for (int k = 0; k < K; ++k)
						{
							const unsigned long long w = ld_relaxed_u64(part + e * 4 + k);
							all = all && uint32_t(w >> 32) == p.tag;
							tot[k] += double(__uint_as_float(uint32_t(w)));
						}
					}
					if (__all_sync(0xffffffffu, all))
					{
						ok = true;
						break;
					}
					if ((round & 63) == 63 && *reinterpret_cast<volatile int *>(&p.report->status) != 0)
						break;
					__nanosleep(200);
				}
				#pragma unroll
				for (int k = 0; k < K; ++k)
					tot[k] = chain_warp_sum(tot[k]);
				if (!ok && lane == 0)
				{
					p.report->status = 4;
					if (p.error_word) *p.error_word = 4;
				}
				// this rank's sums as the other entry points define them: {sum x, sum x^2} forward (the deposits are taken
				// around the channel's first element, undone here in double), {sum du, sum du*xhat, sum slope terms} backward
				float m0, m1, m2 = 0.0F;
				const float saved_mean = BWD ? __ldg(p.saved + ch) : 0.0F, saved_invstd = BWD ? __ldg(p.saved + p.c + ch) : 0.0F;
				const double shift = BWD ? 0.0 : double(__ldg(p.x + size_t(ch) * p.hw));
				if (!BWD)
				{
					m0 = float(tot[0] + p.count * shift);
					m1 = float(tot[1] + 2.0 * shift * tot[0] + p.count * shift * shift);
				}
				else
				{
					m0 = float(tot[0]);
					m1 = float(tot[1] * double(saved_invstd));
					m2 = float(tot[2]);
				}
				double mean_d = 0.0, var_d = 0.0;   // forward
				float c2 = 0.0F, c3 = 0.0F;          // backward
				if (!PEER)
				{
					if (!BWD)
					{
						const double ms = tot[0] / p.count;
						mean_d = shift + ms;
						var_d = tot[1] / p.count - ms * ms;
					}
					else
					{
						c2 = float(double(m0) / p.count);
						c3 = float(double(m1) / p.count);
					}
				}
				else
				{
					// publish this rank's two sums to every rank, wait (bounded) for the words of all ranks, add in rank order
					if (lane < uint32_t(p.world) * 2)
					{
						const uint32_t r = lane >> 1, k = lane & 1;
						st_sys_u64(p.mail[r] + mail_index(p, p.rank, ch) + k, (static_cast<unsigned long long>(p.seq) << 32) | __float_as_uint(k ? m1 : m0));
					}
					const unsigned long long * mine = p.mail[p.rank];
					unsigned long long w0 = 0, w1 = 0;
					bool have = lane >= uint32_t(p.world);
					const unsigned long long t1 = chain_timer_ns();
					for (uint32_t round = 0; ; ++round)
					{
						if (!have)
						{
							w0 = ld_sys_u64(mine + mail_index(p, lane, ch));
							w1 = ld_sys_u64(mine + mail_index(p, lane, ch) + 1);
							have = uint32_t(w0 >> 32) == p.seq && uint32_t(w1 >> 32) == p.seq;
						}
						if (__all_sync(0xffffffffu, have))
							break;
						bool give_up = false;
						if ((round & 15) == 15 && lane == 0)
							give_up = *reinterpret_cast<volatile int *>(&p.report->status) != 0 || chain_timer_ns() - t1 > p.wait_limit_ns;
						if (__any_sync(0xffffffffu, give_up))
						{
							if (lane == 0)
							{
								p.report->status = 2;
								if (p.error_word) *p.error_word = 2;
							}
							break;
						}
						__nanosleep(200);
					}
					float f0 = 0.0F, f1 = 0.0F;
					for (int r = 0; r < p.world; ++r)
					{
						f0 += __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, w0, r)));
						f1 += __uint_as_float(uint32_t(__shfl_sync(0xffffffffu, w1, r)));
					}
					if (!BWD)
					{
						mean_d = double(f0) / p.count_total;
						var_d = double(f1) / p.count_total - mean_d * mean_d;
					}
					else
					{
						c2 = float(double(f0) / p.count_total);
						c3 = float(double(f1) / p.count_total);
					}
				}
				if (lane == 0)
				{
					const unsigned long long waited = chain_timer_ns() - t0;
					atomicAdd(&p.report->wait_ns_total, waited);
					atomicMax(&p.report->wait_ns_max, waited);
					float4 f0v, f1v = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					if (!BWD)
					{
						var_d = var_d < 0.0 ? 0.0 : var_d;
						const float fmean = float(mean_d);
						const float finv = float(1.0 / sqrt(var_d + double(p.eps)));
						const float mult = __ldg(p.gamma + ch) * finv;
						f0v = make_float4(mult, fmaf(-mult, fmean, __ldg(p.beta + ch)), 0.0F, 0.0F);
						p.saved[ch] = fmean;
						p.saved[p.c + ch] = finv;
						if (p.sums)
						{
							p.sums[ch] = m0;
							p.sums[p.c + ch] = m1;
						}
					}
					else
					{
						const float mult = __ldg(p.gamma + ch) * saved_invstd;
						// dx = mult * ((du - c2) - xhat * c3) with xhat = (x - mean) * invstd, as two fused multiply-adds
						f0v = make_float4(mult, -(mult * c3 * saved_invstd), -(mult * c2), saved_mean);
						f1v = make_float4(__ldg(p.beta + ch), 0.0F, 0.0F, 0.0F);
						if (p.sums)
						{
							p.sums[ch] = m0;
							p.sums[p.c + ch] = m1;
							p.sums[2 * p.c + ch] = m2;
						}
						// per-channel gradients accumulate this rank's sums (batch_norm_layer_updater_cuda.cu:138-139, 167-182)
						if (p.grad_beta) p.grad_beta[ch] += m0;
						if (p.grad_gamma) p.grad_gamma[ch] += m1;
						if (p.grad_slope) p.grad_slope[ch] += m2;
						if (p.grad_mean) p.grad_mean[ch] += p.entry_count * (saved_mean - p.mean[ch]);
						if (p.grad_invsigma) p.grad_invsigma[ch] += p.entry_count * (saved_invstd - p.invsigma[ch]);
					}
					p.fin[2 * ch] = f0v;
					p.fin[2 * ch + 1] = f1v;
					st_release_u32(p.ready + ch, 1u);
				}
				return;
			}

			// ---- this thread's slots: fixed byte offsets inside a sweep ------------------------------------
			const uint32_t rows = p.rows, cols = p.cols, tiles = p.tiles;
			const uint32_t entry_stride_b = p.c * p.hw * 4;
			const uint32_t per_item = kind == 0 ? p.es : p.ea;
			const uint32_t e0 = sp * per_item;
			const uint32_t e1 = min(e0 + per_item, p.n);
			const uint32_t nrows = e1 > e0 ? e1 - e0 : 0;
			const uint32_t row_sweeps = p.d_rows.div(nrows + rows - 1);
			const uint32_t rem_rows = nrows - (row_sweeps ? row_sweeps - 1 : 0) * rows;   // rows of the last row sweep
			const uint32_t last_cols = p.vpp - (tiles - 1) * cols;                         // vectors of the last column tile
			uint32_t ob[L];
			uint32_t m_slots = 0, m_rows = 0, m_cols = 0;   // bit u: slot u exists / lies in the last row sweep's rows / in the last column tile
			#pragma unroll
			for (int u = 0; u < L; ++u)
			{
				const uint32_t s = threadIdx.x + u * kChainThreads;
				const uint32_t r = p.d_cols.div(s);
				const uint32_t cidx = s - r * cols;
				ob[u] = r * entry_stride_b + cidx * 16;
				m_slots |= (r < rows ? 1u : 0u) << u;
				m_rows |= (r < rem_rows ? 1u : 0u) << u;
				m_cols |= (cidx < last_cols ? 1u : 0u) << u;
			}
			const uint32_t row_step_b = rows * entry_stride_b;
			const size_t off0 = (size_t(e0) * p.c + ch) * p.hw;
			auto sweep_mask = [&](uint32_t rs, uint32_t ct) -> uint32_t
			{
				uint32_t m = rs < row_sweeps ? m_slots : 0u;
				if (rs + 1 == row_sweeps) m &= m_rows;
				if (ct + 1 == tiles) m &= m_cols;
				return m;
			};
			float4 * const my = ring + threadIdx.x;
			auto slot = [&](int g, int t, int u) -> float4 * { return my + ((g * T + t) * L + u) * kChainThreads; };
			const float slope = chain_slope(p.chain, ch);

			if (kind == 0)
			{
				// ---- S item --------------------------------------------------------------------------
				uint64_t policy;
				asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
				float acc[K];
				#pragma unroll
				for (int k = 0; k < K; ++k)
					acc[k] = 0.0F;
				uint32_t irs = 0, ict = 0, icoff = 0;    // the next sweep to ask for
				const char * ibx = reinterpret_cast<const char *>(p.x + off0);
				const char * ibd = reinterpret_cast<const char *>(BWD ? p.dy + off0 : p.x + off0);
				auto issue = [&](int g)
				{
					if (irs < row_sweeps)
					{
						const uint32_t m = sweep_mask(irs, ict);
						#pragma unroll
						for (int u = 0; u < L; ++u)
							if (m & (1u << u))
							{
								cp_async16(slot(g, 0, u), ibx + icoff + ob[u], policy);
								if (BWD) cp_async16(slot(g, T - 1, u), ibd + icoff + ob[u], policy);
							}
						icoff += cols * 16;
						if (++ict == tiles)
						{
							ict = 0; icoff = 0; ++irs;
							ibx += row_step_b; ibd += row_step_b;
						}
					}
					cp_async_commit();
				};
				#pragma unroll
				for (int g = 0; g < STAGES; ++g)
					issue(g);
				// forward: the sums are taken around the channel's first element, so that a mean far from zero costs no digits
				const float shift = BWD ? 0.0F : __ldg(p.x + size_t(ch) * p.hw);
				const float mean = BWD ? __ldg(p.saved + ch) : 0.0F;
				const float mult = BWD ? __ldg(p.gamma + ch) * __ldg(p.saved + p.c + ch) : 0.0F;
				const float beta = BWD ? __ldg(p.beta + ch) : 0.0F;
				uint32_t crs = 0, cct = 0;
				int g = 0;
				while (row_sweeps)
				{
					cp_async_wait<STAGES - 1>();
					const uint32_t m = sweep_mask(crs, cct);
					#pragma unroll
					for (int u = 0; u < L; ++u)
					{
						if (!(m & (1u << u)))
							continue;
						const float4 a = *slot(g, 0, u);
						if (!BWD)
						{
							const float v0 = a.x - shift, v1 = a.y - shift, v2 = a.z - shift, v3 = a.w - shift;
							acc[0] += (v0 + v1) + (v2 + v3);
							acc[1] = fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, fmaf(v3, v3, acc[1]))));
						}
						else
						{
							const float4 d = *slot(g, T - 1, u);
							const float xs[4] = {a.x, a.y, a.z, a.w};
							const float ds[4] = {d.x, d.y, d.z, d.w};
							#pragma unroll
							for (int j = 0; j < 4; ++j)
							{
								const float xc = xs[j] - mean;
								const float uu = fmaf(xc, mult, beta);
								float term;
								const float du = stream_backward<A0, A1>(p.chain, uu, ds[j], slope, term);
								acc[0] += du;
								acc[1] = fmaf(du, xc, acc[1]);
								acc[K - 1] += term;
							}
						}
					}
					if (++cct == tiles)
					{
						cct = 0;
						if (++crs == row_sweeps)
							break;
					}
					issue(g);
					if (++g == STAGES) g = 0;
				}
				cp_async_wait<0>();
				// the item's deposit: warp sums, then the warps' sums in warp order; each sum travels with the launch's tag
				#pragma unroll
				for (int k = 0; k < K; ++k)
					acc[k] = stream_warp_sum(acc[k]);
				if (lane == 0)
				{
					#pragma unroll
					for (int k = 0; k < K; ++k)
						s_sum[warp][k] = acc[k];
				}
				__syncthreads();
				if (threadIdx.x < K)
				{
					float t = 0.0F;
					#pragma unroll
					for (int w = 0; w < kStreamWarps; ++w)
						t += s_sum[w][threadIdx.x];
					st_relaxed_u64(p.deposit + (size_t(ch) * p.ss + sp) * 4 + threadIdx.x, (static_cast<unsigned long long>(p.tag) << 32) | __float_as_uint(t));
				}
				return;
			}

			// ---- A item ------------------------------------------------------------------------------
			uint64_t policy;
			asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
			uint32_t irs = 0, ict = 0, icoff = 0;
			const char * ibx = reinterpret_cast<const char *>(p.x + off0);
			const char * ibd = reinterpret_cast<const char *>(BWD ? p.dy + off0 : p.x + off0);
			char * bo = reinterpret_cast<char *>(p.out + off0);
			auto issue = [&](int g)
			{
				if (irs < row_sweeps)
				{
					const uint32_t m = sweep_mask(irs, ict);
					#pragma unroll
					for (int u = 0; u < L; ++u)
						if (m & (1u << u))
						{
							cp_async16(slot(g, 0, u), ibx + icoff + ob[u], policy);
							if (BWD) cp_async16(slot(g, T - 1, u), ibd + icoff + ob[u], policy);
						}
					icoff += cols * 16;
					if (++ict == tiles)
					{
						ict = 0; icoff = 0; ++irs;
						ibx += row_step_b; ibd += row_step_b;
					}
				}
				cp_async_commit();
			};
			// the first copies do not depend on the statistics: they are on their way while the item waits
			#pragma unroll
			for (int g = 0; g < STAGES; ++g)
				issue(g);
			if (threadIdx.x == 0)
			{
				bool ok = false;
				unsigned long long t0 = 0;
				for (uint32_t round = 0; round < kChainPollLimit; ++round)
				{
					if (ld_acquire(p.ready + ch) != 0)
					{
						ok = true;
						break;
					}
					if (round == 0)
						t0 = chain_timer_ns();
					if ((round & 63) == 63 && *reinterpret_cast<volatile int *>(&p.report->status) != 0)
						break;
					__nanosleep(100);
				}
				if (t0)
				{
					const unsigned long long waited = chain_timer_ns() - t0;
					atomicAdd(&p.report->wait_ns_total, waited);
					atomicMax(&p.report->wait_ns_max, waited);
				}
				if (!ok && p.report->status == 0)
				{
					p.report->status = 4;
					if (p.error_word) *p.error_word = 4;
				}
				s_fin[0] = __ldcg(p.fin + 2 * ch);
				s_fin[1] = __ldcg(p.fin + 2 * ch + 1);
			}
			__syncthreads();
			const float4 f0 = s_fin[0];
			const float4 f1 = s_fin[1];
			uint32_t crs = 0, cct = 0, coff = 0;
			int g = 0;
			while (row_sweeps)
			{
				cp_async_wait<STAGES - 1>();
				const uint32_t m = sweep_mask(crs, cct);
				#pragma unroll
				for (int u = 0; u < L; ++u)
				{
					if (!(m & (1u << u)))
						continue;
					const float4 a = *slot(g, 0, u);
					float4 o;
					if (!BWD)
					{
						o.x = chain_forward<A0, A1>(p.chain, fmaf(a.x, f0.x, f0.y), slope);
						o.y = chain_forward<A0, A1>(p.chain, fmaf(a.y, f0.x, f0.y), slope);
						o.z = chain_forward<A0, A1>(p.chain, fmaf(a.z, f0.x, f0.y), slope);
						o.w = chain_forward<A0, A1>(p.chain, fmaf(a.w, f0.x, f0.y), slope);
					}
					else
					{
						const float4 d = *slot(g, T - 1, u);
						const float xs[4] = {a.x, a.y, a.z, a.w};
						const float ds[4] = {d.x, d.y, d.z, d.w};
						float r_[4];
						#pragma unroll
						for (int j = 0; j < 4; ++j)
						{
							const float xc = xs[j] - f0.w;
							const float uu = fmaf(xc, f0.x, f1.x);
							float term;
							const float du = stream_backward<A0, A1>(p.chain, uu, ds[j], slope, term);
							r_[j] = fmaf(du, f0.x, fmaf(xc, f0.y, f0.z));
						}
						o = make_float4(r_[0], r_[1], r_[2], r_[3]);
					}
					st_stream(reinterpret_cast<float4 *>(bo + coff + ob[u]), o);
				}
				coff += cols * 16;
				if (++cct == tiles)
				{
					cct = 0; coff = 0;
					bo += row_step_b;
					if (++crs == row_sweeps)
						break;
				}
				issue(g);
				if (++g == STAGES) g = 0;
			}
			cp_async_wait<0>();
		}

		// ---- the same single launch for planes that are not whole float4s (7x7, 13x13) ----------------------------
		// Items are numbered by channel GROUP: 4 / gcd(H*W, 4) adjacent channels of one entry form an aligned run of
		// whole vectors, a group is as many of those as fill the CTA's 256 vector lanes (20 channels for 7x7). A thread
		// owns one vector position of the group's run in every entry of its item, so the channels of its four
		// elements and their constants are loop invariants; an S item sums per position and folds the positions per
		// channel through shared memory; the S item that finishes a group last folds the items' partial sums of all the
		// group's channels and leaves the constants for the group's A items.
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
					// the sums are taken around each channel's first element (undone in double where they are folded), so that a
					// mean far from zero costs no digits of the variance
					float shift[4];
					#pragma unroll
					for (int j = 0; j < 4; ++j)
						shift[j] = __ldg(p.x + size_t(ch0 + local[j]) * p.hw);
					const float4 * bx = reinterpret_cast<const float4 *>(p.x) + base4;
					for (uint32_t e = e0; e < e1; e += U)
					{
						float4 a[U];
						#pragma unroll
						for (int u = 0; u < U; ++u)
						{
							a[u] = make_float4(shift[0], shift[1], shift[2], shift[3]);
							if (active && e + u < e1)
								a[u] = __ldg(bx + size_t(e + u - e0) * stride4); // default policy: stays in L2
						}
						#pragma unroll
						for (int u = 0; u < U; ++u)
						{
							const float v0 = a[u].x - shift[0], v1 = a[u].y - shift[1], v2 = a[u].z - shift[2], v3 = a[u].w - shift[3];
							acc[0][0] += v0; acc[0][1] += v1; acc[0][2] += v2; acc[0][3] += v3;
							acc[1][0] = fmaf(v0, v0, acc[1][0]); acc[1][1] = fmaf(v1, v1, acc[1][1]);
							acc[1][2] = fmaf(v2, v2, acc[1][2]); acc[1][3] = fmaf(v3, v3, acc[1][3]);
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
					}
				}
				__syncthreads();
				if (threadIdx.x == 0)
				{
					// the barrier orders every partial sum of this item, whichever thread wrote it, before this fence, and
					// the fence before the count
					__threadfence();
					const uint32_t before = atomicAdd(p.done + grp, 1u);
					const bool last = before == p.split_s - 1;
					if (last)
						__threadfence(); // the other items' partial sums are visible to the group's last item
					s_item[3] = last ? 1u : 0u;
				}
				__syncthreads();
				if (s_item[3] == 0)
					return;
				// last S item of this group on this rank: fold the partial sums of every channel of the group (slice
				// order, eight lanes per channel) and write the local per-channel outputs. One GPU: derive the constants
				// the group's A items apply and raise the group's flag. Several: publish the messages to every rank.
				for (uint32_t first = 0; first < channels; first += kChainThreads / kLanes)
				{
					const uint32_t lc = first + threadIdx.x / kLanes;
					const uint32_t ch = ch0 + lc;
					double t[K];
					#pragma unroll
					for (int k = 0; k < K; ++k)
						t[k] = 0.0;
					if (lc < channels)
					{
						#pragma unroll 4
						for (uint32_t q = lane; q < p.split_s; q += kLanes)
						{
							#pragma unroll
							for (int k = 0; k < K; ++k)
								t[k] += __ldcg(p.partial + (size_t(ch) * p.split_s + q) * 3 + k);
						}
					}
					#pragma unroll
					for (int k = 0; k < K; ++k)
					{
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 4);
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 2);
						t[k] += __shfl_xor_sync(0xffffffffu, t[k], 1);
					}
					if constexpr (!PEER)
					{
						if (lc < channels && lane == 0)
						{
							float * fin = p.fin + size_t(ch) * 8;
							if constexpr (!BWD)
							{
								const double sh = double(__ldg(p.x + size_t(ch) * p.hw));
								const double ms = t[0] / p.count;       // mean of x - shift
								double var = t[1] / p.count - ms * ms;
								var = var < 0.0 ? 0.0 : var;
								const float fmean = float(sh + ms);
								t[1] = t[1] + 2.0 * sh * t[0] + p.count * sh * sh;   // {sum x, sum x^2} as the other entry points define them
								t[0] = t[0] + p.count * sh;
								const float finv = float(1.0 / sqrt(var + double(p.eps)));
								const float mult = __fmul_rn(__ldg(p.gamma + ch), finv);
								__stcg(reinterpret_cast<float2 *>(fin), make_float2(mult, __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, fmean))));
								p.saved[ch] = fmean;
								p.saved[p.c + ch] = finv;
								if (p.sums)
								{
									p.sums[ch] = float(t[0]);
									p.sums[p.c + ch] = float(t[1]);
								}
							}
							else
							{
								const float fb = float(t[0]), fg = float(t[1]), fs = float(t[K - 1]);
								const float mean = __ldg(p.saved + ch), invstd = __ldg(p.saved + p.c + ch);
								const float mult = __fmul_rn(__ldg(p.gamma + ch), invstd);
								// the same float-rounded sums the two-kernel form passes between its kernels
								__stcg(reinterpret_cast<float4 *>(fin), make_float4(mult, __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean)), mean, invstd));
								__stcg(reinterpret_cast<float2 *>(fin + 4), make_float2(float(double(fb) / p.count), float(double(fg) / p.count)));
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
					else if (lc < channels)
					{
						if constexpr (!BWD)
						{
							// back to {sum x, sum x^2}, the message the ranks exchange
							const double sh = double(__ldg(p.x + size_t(ch) * p.hw));
							const double s0 = t[0];
							t[0] = s0 + p.count * sh;
							t[1] = t[1] + 2.0 * sh * s0 + p.count * sh * sh;
						}
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
				if constexpr (!PEER)
				{
					// the barrier orders the constants, whichever thread wrote them, before the release that raises the flag
					__syncthreads();
					if (threadIdx.x == 0)
						st_release_u32(p.done + p.groups + grp, 1u);
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
							give_up = (p.error && *reinterpret_cast<volatile int *>(p.error) != 0) || chain_timer_ns() - t0 > p.wait_limit_ns;
						if (__any_sync(0xffffffffu, give_up))
						{
							if ((threadIdx.x & 31) == 0 && p.error)
							{
								*p.error = 2;
								if (p.error_word) *p.error_word = 2;
							}
							break;
						}
						__nanosleep(200);
					}
					if ((threadIdx.x & 31) == 0 && p.wait_ns)
					{
						const unsigned long long waited = chain_timer_ns() - t0;
						atomicAdd(p.wait_ns, waited);
						atomicMax(p.wait_ns + 1, waited);
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
				// the flag the group's last S item raises behind the constants
				bool ready = false;
				for (uint32_t round = 0; round < kChainPollLimit; ++round)
				{
					if (ld_acquire(p.done + p.groups + grp) != 0)
					{
						ready = true;
						break;
					}
					__nanosleep(200);
				}
				if (!ready && p.error)
				{
					*p.error = 4;
					if (p.error_word) *p.error_word = 4;
				}
			}
			if constexpr (!PEER)
			{
				__syncthreads();
				for (uint32_t lc = threadIdx.x; lc < channels; lc += kChainThreads)
				{
					const float * fin = p.fin + size_t(ch0 + lc) * 8;
					if constexpr (!BWD)
					{
						const float2 q = __ldcg(reinterpret_cast<const float2 *>(fin));
						s_const[0][lc] = q.x;
						s_const[1][lc] = q.y;
					}
					else
					{
						const float4 q = __ldcg(reinterpret_cast<const float4 *>(fin));
						const float2 r = __ldcg(reinterpret_cast<const float2 *>(fin + 4));
						s_const[0][lc] = q.x;
						s_const[1][lc] = q.y;
						s_const[NC - 4][lc] = q.z;
						s_const[NC - 3][lc] = q.w;
						s_const[NC - 2][lc] = r.x;
						s_const[NC - 1][lc] = r.y;
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

		// Geometry of the kernel for planes of whole float4s. Defaults measured on B200 with x[256,256,28,28],
		// PReLU+ELU (forward / backward): items of 48 KB (statistics) and 64 KB (apply) of one tensor, apply items 32 /
		// 24 channels behind the statistics items: 86 / 150 us. Shorter distances make every apply item wait for its
		// channel (16 channels: 94 / 164 us), longer ones push the first read out of L2 before the second.
		// Knobs: chain_s_kb, chain_a_kb, chain_dist (nnf_set_tuning).
		bool plan_stream(stream_params& p, int64_t n, int64_t c, int64_t hw, bool backward, bool sharded = false)
		{
			if (hw % 4 != 0 || n < 1 || c < 1 || n * hw >= (int64_t(1) << 31) || c > 0x7fffffff / 256)
				return false;
			const int64_t vpp = hw / 4;
			const int64_t slots = int64_t(kChainThreads) * (backward ? kStreamSlotsBwd : kStreamSlots);
			int64_t rows, cols, tiles;
			if (vpp <= slots) { cols = vpp; rows = slots / vpp; tiles = 1; }
			else { cols = slots; rows = 1; tiles = div_up(vpp, slots); }
			if (rows > n) rows = n;
			// slot offsets inside a sweep and the step between sweeps are kept in 32 bits
			if (rows * c * hw * 4 >= (int64_t(1) << 32))
				return false;
			const int64_t plane_bytes = hw * 4;
			auto entries = [&](int kb)
			{
				int64_t e = int64_t(kb) * 1024 / plane_bytes;
				e = e / rows * rows;
				if (e < rows) e = rows;
				if (e > n) e = n;
				return e;
			};
			const tuning& t = tune();
			int64_t es = entries(t.chain_s_kb > 0 ? t.chain_s_kb : 48), ea = entries(t.chain_a_kb > 0 ? t.chain_a_kb : 64);
			if (div_up(n, es) > kChainMaxSplit)
				es = div_up(div_up(n, kChainMaxSplit), rows) * rows;
			if (div_up(n, ea) > 4096)
				ea = div_up(div_up(n, 4096), rows) * rows;
			p.es = (uint32_t)es; p.ea = (uint32_t)ea;
			p.ss = (uint32_t)div_up(n, es); p.sa = (uint32_t)div_up(n, ea);
			// batch-sharded launches: a channel's constants also wait for the other ranks' sums (an NVLink round trip and whatever
			// the ranks are apart), so the forward launch keeps a longer distance (two GPUs, before the staging ring: 119 us at
			// 48 against 127-130 at 32; with it 88 us at either)
			int64_t dist = t.chain_dist >= 0 ? t.chain_dist : (backward ? 24 : (sharded ? 48 : 32));
			if (dist > c) dist = c;
			p.dist = (uint32_t)dist;
			p.dist_f = (uint32_t)(dist / 2);
			const int64_t total = (c + dist) * (int64_t(p.ss) + p.sa + 1);
			if (total >= (int64_t(1) << 31))
				return false;
			p.total = (uint32_t)total;
			p.n = (uint32_t)n; p.c = (uint32_t)c; p.hw = (uint32_t)hw; p.vpp = (uint32_t)vpp;
			p.rows = (uint32_t)rows; p.cols = (uint32_t)cols; p.tiles = (uint32_t)tiles;
			p.d_cols = fastdiv(p.cols); p.d_per = fastdiv(p.ss + p.sa + 1); p.d_both = fastdiv(p.ss + p.sa); p.d_rows = fastdiv(p.rows);
			p.count = double(n) * double(hw);
			return true;
		}

		size_t stream_workspace_needed(const stream_params& p)
		{
			return sizeof(launch_report) + size_t(p.c) * sizeof(uint32_t) + 16 + size_t(p.c) * 2 * sizeof(float4)
				+ size_t(p.c) * p.ss * 4 * sizeof(unsigned long long);
		}

		// The grouped kernel's plan: items are channel groups. Returns false where the shape does not suit it (planes
		// of whole float4s take the kernel above; runs shorter than 16 vectors or longer than 256 the separate kernels).
		bool plan_chain_grouped(chain_params& p, int64_t n, int64_t c, int64_t hw, bool backward = false)
		{
			if (hw % 4 == 0 || n < 1 || c < 1 || n >= (int64_t(1) << 31) || c >= (int64_t(1) << 24) || tune().no_grouped == 1)
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
			const int64_t s_bytes = int64_t(tune().chain_s_kb > 0 ? tune().chain_s_kb : 48) * 1024;
			const int64_t a_bytes = int64_t(tune().chain_a_kb > 0 ? tune().chain_a_kb : 64) * 1024;
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
			int64_t chunk = (int64_t)(double(tune().chain_chunk_mb > 0 ? tune().chain_chunk_mb : 16) * 1024.0 * 1024.0 / group_bytes);
			if (chunk < 1) chunk = 1;
			if (chunk < div_up(groups, 64)) chunk = div_up(groups, 64);
			if (chunk > groups) chunk = groups;
			p.chunk = (uint32_t)chunk;
			p.nchunks = (uint32_t)div_up(groups, chunk);
			// the knob is lag + 1, so that 0 keeps the default: two chunks forward, one backward (x[1024,512,7,7] with ReLU on
			// B200: forward 62 us at one chunk, 58 us at two; backward 90 us and 91 us)
			int lag = tune().chain_lag > 0 ? tune().chain_lag - 1 : (backward ? 1 : 2);
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

		// Workspace of the channel-group kernel: the report, the counters (one per channel + padding), the partial sums,
		// eight floats of constants per channel (16-byte aligned).
		size_t chain_workspace_needed(const chain_params& p)
		{
			return sizeof(launch_report) + (size_t(p.c) + 2) / 2 * 2 * sizeof(uint32_t) + size_t(p.c) * p.split_s * 3 * sizeof(double) + 16 + size_t(p.c) * 8 * sizeof(float);
		}

		unsigned long long peer_wait_limit()
		{
			const long long v = tune().peer_wait_ns;
			return v > 0 ? (unsigned long long)v : kDefaultPeerWaitNs;
		}

		template <class Kernel>
		int launch_chain(Kernel kernel, chain_params& p, void * workspace, cudaStream_t s, const char * what)
		{
			launch_report * report = static_cast<launch_report *>(workspace);
			p.done = reinterpret_cast<uint32_t *>(report + 1);
			p.partial = reinterpret_cast<double *>(p.done + (size_t(p.c) + 2) / 2 * 2);
			p.fin = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(p.partial + size_t(p.c) * p.split_s * 3) + 15) & ~uintptr_t(15));
			p.ticket = &report->ticket;
			p.error = &report->status;
			p.wait_ns = &report->wait_ns_total;
			p.error_word = device_error_word();
			p.wait_limit_ns = peer_wait_limit();
			cudaError_t e = cudaMemsetAsync(workspace, 0, sizeof(launch_report) + size_t(p.c) * sizeof(uint32_t), s);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s: cudaMemsetAsync: %s", what, cudaGetErrorString(e));
			kernel<<<p.total_items, kChainThreads, 0, s>>>(p);
			return check_launch(what);
		}

		std::atomic<uint32_t> g_launch_tag{0};

		template <class Kernel>
		int launch_stream(Kernel kernel, stream_params& p, void * workspace, cudaStream_t s, bool backward, const char * what)
		{
			launch_report * report = static_cast<launch_report *>(workspace);
			p.report = report;
			p.ready = reinterpret_cast<uint32_t *>(report + 1);
			char * after = reinterpret_cast<char *>(p.ready) + (size_t(p.c) * sizeof(uint32_t) + 15) / 16 * 16;
			p.fin = reinterpret_cast<float4 *>(after);
			p.deposit = reinterpret_cast<unsigned long long *>(p.fin + size_t(p.c) * 2);
			p.error_word = device_error_word();
			p.wait_limit_ns = peer_wait_limit();
			uint32_t tag = ++g_launch_tag;
			if (tag == 0)
				tag = ++g_launch_tag;   // zero is what a fresh workspace holds
			p.tag = tag;
			const size_t smem = size_t(backward ? kStagesBwd * 2 * kStreamSlotsBwd : kStagesFwd * kStreamSlots) * kChainThreads * sizeof(float4);
			cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
			e = cudaMemsetAsync(workspace, 0, sizeof(launch_report) + size_t(p.c) * sizeof(uint32_t), s);
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "%s: cudaMemsetAsync: %s", what, cudaGetErrorString(e));
			kernel<<<p.total, kChainThreads, smem, s>>>(p);
			return check_launch(what);
		}
	}

	size_t chain_workspace_bytes(int64_t n, int64_t c, int64_t hw)
	{
		// the larger of what the two kernels plan for this shape, forward or backward (the plans share their item counts)
		// the knobs may change between the size query and the launch: sized for the most items a plan can make
		(void)n; (void)hw;
		const size_t grouped = sizeof(launch_report) + (size_t(c) + 2) / 2 * 2 * sizeof(uint32_t) + size_t(c) * kChainMaxSplit * 3 * sizeof(double)
			+ 16 + size_t(c) * 8 * sizeof(float);
		const size_t stream = sizeof(launch_report) + size_t(c) * sizeof(uint32_t) + 16 + size_t(c) * 2 * sizeof(float4)
			+ size_t(c) * kChainMaxSplit * 4 * sizeof(unsigned long long);
		return grouped > stream ? grouped : stream;
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

		template <class Params>
		int fill_peer(Params& p, const chain_peer * peer, const char * who)
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

		bool workspace_ok(const void * workspace, size_t have, size_t need)
		{
			return workspace && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 && have >= need;
		}

		template <bool PEER>
		int chain_forward_impl(cudaStream_t stream, float * y, float * saved, float * sums, const float * x, const float * gamma, const float * beta,
			float eps, const act_chain& chain, int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes, const chain_peer * peer)
		{
			if (!aligned16(x) || !aligned16(y))
				return 1;
			chain_params gp = {};
			if (plan_chain_grouped(gp, n, c, hw))
			{
				if (!workspace_ok(workspace, workspace_bytes, chain_workspace_needed(gp)))
					return 2;
				gp.x = x; gp.out = y; gp.gamma = gamma; gp.beta = beta; gp.saved = saved; gp.sums = sums;
				gp.chain = chain;
				gp.eps = eps;
				const int st = fill_peer(gp, peer, "bn_train_chain_grouped_kernel (forward)");
				if (st != NNF_OK)
					return st;
				const char * what = "bn_train_chain_grouped_kernel (forward)";
				switch (chain_id(chain))
				{
				case 0: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_NONE, 0, false, PEER>, gp, workspace, stream, what);
				case 1: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, false, PEER>, gp, workspace, stream, what);
				case 2: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_RELU, 0, false, PEER>, gp, workspace, stream, what);
				default: return launch_chain(bn_train_chain_grouped_kernel<-1, 0, false, PEER>, gp, workspace, stream, what);
				}
			}
			stream_params p = {};
			if (!plan_stream(p, n, c, hw, false, PEER))
				return 1;
			if (!workspace_ok(workspace, workspace_bytes, stream_workspace_needed(p)))
				return 2;
			p.x = x; p.out = y; p.gamma = gamma; p.beta = beta; p.saved = saved; p.sums = sums;
			p.chain = chain;
			p.eps = eps;
			const char * what = "bn_train_chain_kernel (forward)";
			const int st = fill_peer(p, peer, what);
			if (st != NNF_OK)
				return st;
			switch (chain_id(chain))
			{
			case 0: return launch_stream(bn_train_chain_kernel<NNF_ACT_NONE, 0, false, PEER>, p, workspace, stream, false, what);
			case 1: return launch_stream(bn_train_chain_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, false, PEER>, p, workspace, stream, false, what);
			case 2: return launch_stream(bn_train_chain_kernel<NNF_ACT_RELU, 0, false, PEER>, p, workspace, stream, false, what);
			default: return launch_stream(bn_train_chain_kernel<-1, 0, false, PEER>, p, workspace, stream, false, what);
			}
		}

		template <bool PEER>
		int chain_backward_impl(cudaStream_t stream, float * dx, float * bsums, const float * dy, const float * x,
			const float * gamma, const float * beta, const float * saved, const act_chain& chain,
			float * grad_gamma, float * grad_beta, float * grad_mean, float * grad_invsigma, float * grad_slope,
			const float * mean, const float * invsigma, float entry_count,
			int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes, const chain_peer * peer)
		{
			if (!aligned16(x) || !aligned16(dy) || !aligned16(dx))
				return 1;
			chain_params gp = {};
			if (plan_chain_grouped(gp, n, c, hw, true))
			{
				if (!workspace_ok(workspace, workspace_bytes, chain_workspace_needed(gp)))
					return 2;
				gp.x = x; gp.dy = dy; gp.out = dx; gp.gamma = gamma; gp.beta = beta; gp.saved = const_cast<float *>(saved); gp.sums = bsums;
				gp.grad_gamma = grad_gamma; gp.grad_beta = grad_beta; gp.grad_mean = grad_mean; gp.grad_invsigma = grad_invsigma; gp.grad_slope = grad_slope;
				gp.mean = mean; gp.invsigma = invsigma; gp.entry_count = entry_count;
				gp.chain = chain;
				const int st = fill_peer(gp, peer, "bn_train_chain_grouped_kernel (backward)");
				if (st != NNF_OK)
					return st;
				const char * what = "bn_train_chain_grouped_kernel (backward)";
				switch (chain_id(chain))
				{
				case 0: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_NONE, 0, true, PEER>, gp, workspace, stream, what);
				case 1: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, true, PEER>, gp, workspace, stream, what);
				case 2: return launch_chain(bn_train_chain_grouped_kernel<NNF_ACT_RELU, 0, true, PEER>, gp, workspace, stream, what);
				default: return launch_chain(bn_train_chain_grouped_kernel<-1, 0, true, PEER>, gp, workspace, stream, what);
				}
			}
			stream_params p = {};
			if (!plan_stream(p, n, c, hw, true, PEER))
				return 1;
			if (!workspace_ok(workspace, workspace_bytes, stream_workspace_needed(p)))
				return 2;
			p.x = x; p.dy = dy; p.out = dx; p.gamma = gamma; p.beta = beta; p.saved = const_cast<float *>(saved); p.sums = bsums;
			p.grad_gamma = grad_gamma; p.grad_beta = grad_beta; p.grad_mean = grad_mean; p.grad_invsigma = grad_invsigma; p.grad_slope = grad_slope;
			p.mean = mean; p.invsigma = invsigma; p.entry_count = entry_count;
			p.chain = chain;
			const char * what = "bn_train_chain_kernel (backward)";
			const int st = fill_peer(p, peer, what);
			if (st != NNF_OK)
				return st;
			switch (chain_id(chain))
			{
			case 0: return launch_stream(bn_train_chain_kernel<NNF_ACT_NONE, 0, true, PEER>, p, workspace, stream, true, what);
			case 1: return launch_stream(bn_train_chain_kernel<NNF_ACT_PRELU, NNF_ACT_ELU, true, PEER>, p, workspace, stream, true, what);
			case 2: return launch_stream(bn_train_chain_kernel<NNF_ACT_RELU, 0, true, PEER>, p, workspace, stream, true, what);
			default: return launch_stream(bn_train_chain_kernel<-1, 0, true, PEER>, p, workspace, stream, true, what);
			}
		}
	}

}

using namespace nnf;

extern "C" int nnf_bn_train_sharded_supported(int64_t n, int64_t c, int64_t hw)
{
	chain_params p = {};
	stream_params q = {};
	return (plan_chain_grouped(p, n, c, hw) || plan_stream(q, n, c, hw, false)) ? 1 : 0;
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
	if (st == 2)
		return set_error(NNF_ERR_WORKSPACE, "nnf_bn_train_fwd_sharded: a 16-byte aligned workspace of nnf_bn_train_workspace_bytes() bytes is required");
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
	if (st == 2)
		return set_error(NNF_ERR_WORKSPACE, "nnf_bn_train_bwd_sharded: a 16-byte aligned workspace of nnf_bn_train_workspace_bytes() bytes is required");
	if (st == 1)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_train_bwd_sharded: needs a shape for which nnf_bn_train_sharded_supported() answers 1, 16-byte aligned tensors and a workspace of nnf_bn_train_workspace_bytes()");
	return st;
}

// The library's process-wide error word: a device variable inside the library, so that reaching it needs no
// allocation - or, once the host has handed one over with nnf_set_error_sink, a word in host memory that the device can
// address (pinned memory), which the host then reads without a copy, an event or a synchronisation. Kernels raise it next
// to their launch's own status word; no kernel reads it, so an old failure cannot make a later launch give up its waits.
static __device__ int nnf_error_word_storage;
static std::atomic<int *> nnf_error_sink{nullptr};

namespace nnf
{
	int * device_error_word()
	{
		if (int * sink = nnf_error_sink.load(std::memory_order_acquire))
			return sink;
		static std::mutex mu;
		static int * words[64] = {};
		int dev = 0;
		if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
			return nullptr;
		std::lock_guard<std::mutex> lock(mu);
		if (!words[dev])
		{
			int * w = nullptr;
			if (cudaGetSymbolAddress((void **)&w, nnf_error_word_storage) != cudaSuccess)
			{
				cudaGetLastError();
				return nullptr;
			}
			words[dev] = w;
		}
		return words[dev];
	}
}

extern "C" int nnf_set_error_sink(int32_t * host_visible_word)
{
	if (host_visible_word)
	{
		cudaPointerAttributes attr;
		if (cudaPointerGetAttributes(&attr, host_visible_word) != cudaSuccess || attr.type != cudaMemoryTypeHost || !attr.devicePointer)
		{
			cudaGetLastError();
			return nnf::set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_set_error_sink: the word must be in pinned host memory that the device can address");
		}
		if (attr.devicePointer != static_cast<void *>(host_visible_word))
			return nnf::set_error(NNF_ERR_UNSUPPORTED, "nnf_set_error_sink: host and device addresses of the word differ (no unified addressing)");
	}
	nnf_error_sink.store(host_visible_word, std::memory_order_release);
	return NNF_OK;
}

// Reads and clears the process-wide error word. With a host-visible sink this is a plain read; otherwise it synchronises the
// device and is meant for tests and diagnosis, not for the enqueue path.
extern "C" int nnf_fused_error_check(void)
{
	if (int * sink = nnf_error_sink.load(std::memory_order_acquire))
	{
		const int v = *static_cast<volatile int *>(sink);
		if (v)
			*static_cast<volatile int *>(sink) = 0;
		return v;
	}
	int * w = nnf::device_error_word();
	if (!w)
		return 0;
	int v = 0;
	if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
		return -1;
	if (v)
		cudaMemset(w, 0, sizeof(int));
	return v;
}

extern "C" int nnf_bn_train_read_report(nnf_stream_t stream, nnf_launch_report * host_report, const void * workspace)
{
	static_assert(sizeof(nnf_launch_report) <= sizeof(launch_report), "the public report is a prefix of the workspace head");
	if (!host_report || !workspace)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_read_report: null pointer");
	const cudaError_t e = cudaMemcpyAsync(host_report, workspace, sizeof(nnf_launch_report), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
	if (e != cudaSuccess)
		return set_error(NNF_ERR_CUDA, "nnf_bn_train_read_report: cudaMemcpyAsync: %s", cudaGetErrorString(e));
	return NNF_OK;
}

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
	st = chain_forward_impl<false>((cudaStream_t)stream, y, saved, sums, x, gamma, beta, eps, chain, n, c, hw, workspace, workspace_bytes, nullptr);
	if (st == 2)
		return set_error(NNF_ERR_WORKSPACE, "nnf_bn_train_fwd: a 16-byte aligned workspace of %zu bytes is required, got %zu",
			nnf_bn_train_workspace_bytes(n, c, hw), workspace_bytes);
	if (st != 1)
		return st;
	// shapes the single launch does not take (unaligned tensors, planes that neither are whole float4s nor fill
	// channel groups, extents beyond its index range): statistics kernel, then apply kernel
	if (!sums)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_train_fwd: this shape needs the two-kernel form, which requires the sums buffer");
	st = nnf_bn_train_stats(stream, sums, x, n, c, hw, workspace, workspace_bytes);
	if (st != NNF_OK)
		return st;
	return nnf_bn_train_apply_act(stream, y, saved, x, gamma, beta, sums, double(n) * double(hw), eps, acts, n_acts, n, c, hw);
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
	if (!add_to_destination)
	{
		st = chain_backward_impl<false>((cudaStream_t)stream, dx, bsums, dy, x, gamma, beta, saved, chain, grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope,
			mean, invsigma, entry_count, n, c, hw, workspace, workspace_bytes, nullptr);
		if (st == 2)
			return set_error(NNF_ERR_WORKSPACE, "nnf_bn_train_bwd: a 16-byte aligned workspace of %zu bytes is required, got %zu",
				nnf_bn_train_workspace_bytes(n, c, hw), workspace_bytes);
		if (st != 1)
			return st;
	}
	// dx accumulated into its destination, or a shape the single launch does not take: two kernels
	st = nnf_bn_train_bwd_stats(stream, bsums, nullptr, dy, x, gamma, beta, saved, acts, n_acts, n, c, hw, workspace, workspace_bytes);
	if (st != NNF_OK)
		return st;
	return nnf_bn_train_bwd_apply(stream, dx, dy, x, gamma, beta, saved, bsums, bsums, double(n) * double(hw), acts, n_acts,
		grad_gamma, grad_beta, grad_mean, grad_invsigma, grad_slope, mean, invsigma, entry_count, n, c, hw, add_to_destination);
}
