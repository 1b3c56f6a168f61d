// Streaming per-element kernels: inference batch norm (+ residual add) (+ activation chain),
// stand-alone activations forward/backward, the add layer. One HBM pass each: every input element is
// read once with a 128-bit streaming load and every output written once with a 128-bit streaming
// store. HBM-bound: algorithmic bytes per element = 4 * (inputs + outputs).
#include "nnf_common.cuh"

#include <stdlib.h>

namespace nnf
{
	namespace
	{
		constexpr int kThreads = 256;
		constexpr int kUnroll = 4;             // independent 128-bit loads in flight per thread and tensor
		constexpr int kCtasPerSm = 8;          // 2048 resident threads per SM
		constexpr int kMaxSmemChannels = 4096; // mult/add staged in shared memory up to this many channels

		struct ew_params
		{
			float * y;
			const float * x;
			const float * res;      // residual (second add input) or null
			const float * gamma;    // null -> no batch norm
			const float * beta;
			const float * mean;
			const float * invsigma;
			const float * sums;     // training mode: {sum x, sum x^2} per channel over all shards; mean/invsigma unused
			float * saved;          // training mode: receives {mean, invstd}
			double count_total;     // training mode: elements per channel over all shards
			float eps;
			float add_alpha;
			uint32_t count;         // elements in this launch (< 2^31)
			uint32_t c;
			fastdiv hw;
			fastdiv cdiv;
			const float * slope;    // the chain's PReLU slopes, or null
			const float * bias;     // per-channel bias added to x first, or null
			int need_channel;       // per-channel parameters are used
			int smem_params;        // mult/add staged in shared memory
			act_chain chain;
		};

		// Per-vector parameters: fetched once per 128-bit vector (MODE 0) or per element (MODE 1/2) and
		// kept in registers, so that the per-element work is only the arithmetic itself.
		struct elem_params
		{
			float mult, add, slope, bias;
		};

		__device__ __forceinline__ elem_params fetch_params(const ew_params& p, const float * s_mult, const float * s_add, uint32_t e)
		{
			elem_params q;
			q.mult = 1.0F; q.add = 0.0F; q.slope = 0.0F; q.bias = 0.0F;
			if (p.need_channel)
			{
				const uint32_t plane = p.hw.div(e);
				const uint32_t channel = plane - p.cdiv.div(plane) * p.c;
				if (p.gamma)
				{
					if (p.smem_params)
					{
						q.mult = s_mult[channel];
						q.add = s_add[channel];
					}
					else
					{
						q.mult = __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel));
						q.add = __fsub_rn(__ldg(p.beta + channel), __fmul_rn(q.mult, __ldg(p.mean + channel)));
					}
				}
				if (p.slope)
					q.slope = __ldg(p.slope + channel);
				if (p.bias)
					q.bias = __ldg(p.bias + channel);
			}
			return q;
		}

		// the per-channel parameters of one channel
		__device__ __forceinline__ elem_params fetch_channel(const ew_params& p, const float * s_mult, const float * s_add, uint32_t channel)
		{
			elem_params q;
			q.mult = 1.0F; q.add = 0.0F; q.slope = 0.0F; q.bias = 0.0F;
			if (p.gamma)
			{
				if (p.smem_params)
				{
					q.mult = s_mult[channel];
					q.add = s_add[channel];
				}
				else
				{
					q.mult = __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel));
					q.add = __fsub_rn(__ldg(p.beta + channel), __fmul_rn(q.mult, __ldg(p.mean + channel)));
				}
			}
			if (p.slope)
				q.slope = __ldg(p.slope + channel);
			if (p.bias)
				q.bias = __ldg(p.bias + channel);
			return q;
		}

		__device__ __forceinline__ elem_params select_params(bool second, const elem_params& a, const elem_params& b)
		{
			elem_params q;
			q.mult = second ? b.mult : a.mult;
			q.add = second ? b.add : a.add;
			q.slope = second ? b.slope : a.slope;
			q.bias = second ? b.bias : a.bias;
			return q;
		}

		// One element: batch norm -> residual add -> activations, in the plain backend's operation order.
		template <int A0, int A1>
		__device__ __forceinline__ float ew_element(const ew_params& p, bool has_bn, bool has_res, const elem_params& q, float x, float r)
		{
			float t = x;
			if (p.bias)
				t = __fadd_rn(t, q.bias); // the producing convolution's bias, added as its own rounded step (cudnnAddTensor after the convolution)
			if (has_bn)
				t = __fadd_rn(__fmul_rn(t, q.mult), q.add); // batch_norm_layer_tester_plain.cpp:70
			if (has_res)
				t = __fmul_rn(__fadd_rn(__fadd_rn(0.0F, t), r), p.add_alpha); // add_layer_tester_plain.cpp:57-60: the accumulator starts at +0.0f
			return chain_forward<A0, A1>(p.chain, t, q.slope);
		}

		// MODE 0: 128-bit accesses, one channel per vector (hw % 4 == 0, or no per-channel parameters)
		// MODE 1: 128-bit accesses, channel derived per element (planes not multiples of 4 elements)
		// MODE 2: scalar accesses (a buffer is not 16-byte aligned)
		template <int MODE, int A0, int A1>
		__global__ void __launch_bounds__(kThreads) bn_act_kernel(const ew_params p)
		{
			extern __shared__ float s_params[];
			float * s_mult = s_params;
			float * s_add = s_params + p.c;
			const bool has_bn = p.gamma != nullptr;
			const bool has_res = p.res != nullptr;
			if (has_bn && p.smem_params && !p.sums)
			{
				// running statistics: four channels per thread in flight (the table is filled once per CTA, and with
				// thousands of channels a chain of dependent loads per channel would cost microseconds)
				for (uint32_t ch0 = threadIdx.x; ch0 < p.c; ch0 += kThreads * 4)
				{
					float g[4], b[4], m[4], is[4];
					#pragma unroll
					for (int u = 0; u < 4; ++u)
					{
						const uint32_t ch = ch0 + u * kThreads;
						if (ch < p.c)
						{
							g[u] = __ldg(p.gamma + ch);
							b[u] = __ldg(p.beta + ch);
							m[u] = __ldg(p.mean + ch);
							is[u] = __ldg(p.invsigma + ch);
						}
					}
					#pragma unroll
					for (int u = 0; u < 4; ++u)
					{
						const uint32_t ch = ch0 + u * kThreads;
						if (ch < p.c)
						{
							// batch_norm_layer_tester_plain.cpp:60-61
							const float mult = __fmul_rn(g[u], is[u]);
							s_mult[ch] = mult;
							s_add[ch] = __fsub_rn(b[u], __fmul_rn(mult, m[u]));
						}
					}
				}
				__syncthreads();
			}
			else if (has_bn && p.smem_params)
			{
				for (uint32_t ch = threadIdx.x; ch < p.c; ch += kThreads)
				{
					float mean, invsigma;
					if (p.sums)
					{
						// batch statistics: biased variance from the (all-reduced) sum and sum of squares
						const double m = double(__ldg(p.sums + ch)) / p.count_total;
						double var = double(__ldg(p.sums + p.c + ch)) / p.count_total - m * m;
						var = var < 0.0 ? 0.0 : var;
						mean = float(m);
						invsigma = float(1.0 / sqrt(var + double(p.eps)));
						if (blockIdx.x == 0 && p.saved)
						{
							p.saved[ch] = mean;
							p.saved[p.c + ch] = invsigma;
						}
					}
					else
					{
						mean = __ldg(p.mean + ch);
						invsigma = __ldg(p.invsigma + ch);
					}
					// batch_norm_layer_tester_plain.cpp:60-61
					const float mult = __fmul_rn(__ldg(p.gamma + ch), invsigma);
					s_mult[ch] = mult;
					s_add[ch] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
				}
				__syncthreads();
			}

			if (MODE == 2)
			{
				const uint32_t stride = gridDim.x * kThreads;
				for (uint32_t e = blockIdx.x * kThreads + threadIdx.x; e < p.count; e += stride)
				{
					const elem_params q = fetch_params(p, s_mult, s_add, e);
					const float r = has_res ? ld_stream(p.res + e) : 0.0F;
					st_stream(p.y + e, ew_element<A0, A1>(p, has_bn, has_res, q, ld_stream(p.x + e), r));
				}
				return;
			}

			const uint32_t nvec = p.count >> 2;
			const float4 * x4 = reinterpret_cast<const float4 *>(p.x);
			const float4 * r4 = reinterpret_cast<const float4 *>(p.res);
			float4 * y4 = reinterpret_cast<float4 *>(p.y);
			const uint32_t tile = kThreads * kUnroll;
			const uint32_t ntiles = (nvec + tile - 1) / tile;

			for (uint32_t t = blockIdx.x; t < ntiles; t += gridDim.x)
			{
				const uint32_t v0 = t * tile + threadIdx.x;
				float4 xv[kUnroll], rv[kUnroll];
				#pragma unroll
				for (int j = 0; j < kUnroll; ++j)
				{
					const uint32_t v = v0 + j * kThreads;
					rv[j] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					if (v < nvec)
					{
						xv[j] = ld_stream(x4 + v);
						if (has_res)
							rv[j] = ld_stream(r4 + v);
					}
				}
				#pragma unroll
				for (int j = 0; j < kUnroll; ++j)
				{
					const uint32_t v = v0 + j * kThreads;
					if (v < nvec)
					{
						const uint32_t e = v << 2;
						float4 o;
						if (MODE == 0)
						{
							const elem_params q = fetch_params(p, s_mult, s_add, e);
							o.x = ew_element<A0, A1>(p, has_bn, has_res, q, xv[j].x, rv[j].x);
							o.y = ew_element<A0, A1>(p, has_bn, has_res, q, xv[j].y, rv[j].y);
							o.z = ew_element<A0, A1>(p, has_bn, has_res, q, xv[j].z, rv[j].z);
							o.w = ew_element<A0, A1>(p, has_bn, has_res, q, xv[j].w, rv[j].w);
						}
						else if (p.hw.d >= 4)
						{
							// planes of at least four elements that are not whole vectors: a vector touches at most two
							// channels, so plane and channel are derived once per vector (two divisions instead of eight)
							// and the parameters of the vector's first channel and of the next are selected per element
							const uint32_t plane = p.hw.div(e);
							const uint32_t left = (plane + 1) * p.hw.d - e;   // elements of the vector's first plane from e on (>= 1)
							const uint32_t channel = plane - p.cdiv.div(plane) * p.c;
							const elem_params qa = fetch_channel(p, s_mult, s_add, channel);
							const elem_params qb = fetch_channel(p, s_mult, s_add, channel + 1 == p.c ? 0 : channel + 1);
							o.x = ew_element<A0, A1>(p, has_bn, has_res, qa, xv[j].x, rv[j].x);
							o.y = ew_element<A0, A1>(p, has_bn, has_res, select_params(left <= 1, qa, qb), xv[j].y, rv[j].y);
							o.z = ew_element<A0, A1>(p, has_bn, has_res, select_params(left <= 2, qa, qb), xv[j].z, rv[j].z);
							o.w = ew_element<A0, A1>(p, has_bn, has_res, select_params(left <= 3, qa, qb), xv[j].w, rv[j].w);
						}
						else
						{
							// planes of one to three elements (fully connected shapes): the channel advances inside the vector
							const uint32_t plane = p.hw.div(e);
							uint32_t pos = e - plane * p.hw.d;
							uint32_t channel = plane - p.cdiv.div(plane) * p.c;
							auto advance = [&]()
							{
								if (++pos == p.hw.d)
								{
									pos = 0;
									channel = channel + 1 == p.c ? 0 : channel + 1;
								}
							};
							o.x = ew_element<A0, A1>(p, has_bn, has_res, fetch_channel(p, s_mult, s_add, channel), xv[j].x, rv[j].x);
							advance();
							o.y = ew_element<A0, A1>(p, has_bn, has_res, fetch_channel(p, s_mult, s_add, channel), xv[j].y, rv[j].y);
							advance();
							o.z = ew_element<A0, A1>(p, has_bn, has_res, fetch_channel(p, s_mult, s_add, channel), xv[j].z, rv[j].z);
							advance();
							o.w = ew_element<A0, A1>(p, has_bn, has_res, fetch_channel(p, s_mult, s_add, channel), xv[j].w, rv[j].w);
						}
						st_stream(y4 + v, o);
					}
				}
			}

			// ragged tail (count % 4 elements), handled by the first threads of the first block
			const uint32_t tail0 = nvec << 2;
			if (blockIdx.x == 0 && tail0 + threadIdx.x < p.count)
			{
				const uint32_t e = tail0 + threadIdx.x;
				const elem_params q = fetch_params(p, s_mult, s_add, e);
				const float r = has_res ? p.res[e] : 0.0F;
				p.y[e] = ew_element<A0, A1>(p, has_bn, has_res, q, p.x[e], r);
			}
		}

		// ---- planes that are not whole float4s (7x7, 13x13): channel groups ---------------------------------------------
		// The flat kernel above must find the channel of every vector by two divisions and fetch two channels'
		// parameters per vector, and stays instruction- and latency-bound on such planes (x[1024,512,7,7] BN+ReLU: 68 % of
		// the copy bandwidth). Here a CTA owns a group of adjacent channels (a multiple of 4 / gcd(H*W, 4), so that the
		// group's run in one entry is aligned and a whole number of vectors; as many as fill the 256 vector lanes: 20 for
		// 7x7) and a slice of entries; a thread owns one vector position of the run in every entry, so the parameters of
		// its four elements are loop invariants in registers and the loop is loads, arithmetic and stores only.
		struct ewg_geom
		{
			uint32_t n, group, groups, split, entries_per_cta;
			uint32_t threads;          // vectors of a full group's run, rounded up to whole warps
			fastdiv d_hw;
		};

		template <int A0, int A1>
		__global__ void __launch_bounds__(kThreads) bn_act_grouped_kernel(const ew_params p, const ewg_geom g)
		{
			extern __shared__ float s_params[];
			float * s_mult = s_params;
			float * s_add = s_params + g.group;
			constexpr int U = 4;   // entries in flight per thread and tensor
			const bool has_bn = p.gamma != nullptr;
			const bool has_res = p.res != nullptr;
			const uint32_t hw = p.hw.d;
			const uint32_t walk = blockIdx.x / g.split;
			const uint32_t sp = blockIdx.x - walk * g.split;
			const uint32_t ch0 = walk * g.group;
			const uint32_t channels = min(g.group, p.c - ch0);
			const uint32_t run = channels * hw;
			const uint32_t v = threadIdx.x;
			const bool active = v < (run >> 2);
			const uint32_t e0 = sp * g.entries_per_cta;
			const uint32_t e1 = min(e0 + g.entries_per_cta, g.n);
			if (has_bn)
			{
				for (uint32_t i = threadIdx.x; i < channels; i += blockDim.x)
				{
					const uint32_t ch = ch0 + i;
					float mean, invsigma;
					if (p.sums)
					{
						// batch statistics: biased variance from the (all-reduced) sum and sum of squares
						const double m = double(__ldg(p.sums + ch)) / p.count_total;
						double var = double(__ldg(p.sums + p.c + ch)) / p.count_total - m * m;
						var = var < 0.0 ? 0.0 : var;
						mean = float(m);
						invsigma = float(1.0 / sqrt(var + double(p.eps)));
						if (sp == 0 && p.saved)
						{
							p.saved[ch] = mean;
							p.saved[p.c + ch] = invsigma;
						}
					}
					else
					{
						mean = __ldg(p.mean + ch);
						invsigma = __ldg(p.invsigma + ch);
					}
					// batch_norm_layer_tester_plain.cpp:60-61
					const float mult = __fmul_rn(__ldg(p.gamma + ch), invsigma);
					s_mult[i] = mult;
					s_add[i] = __fsub_rn(__ldg(p.beta + ch), __fmul_rn(mult, mean));
				}
				__syncthreads();
			}
			if (!active || e0 >= e1)
				return;
			elem_params q[4];
			#pragma unroll
			for (int j = 0; j < 4; ++j)
			{
				const uint32_t local = g.d_hw.div(min(v * 4 + j, run - 1));
				q[j].mult = has_bn ? s_mult[local] : 1.0F;
				q[j].add = has_bn ? s_add[local] : 0.0F;
				q[j].slope = p.slope ? __ldg(p.slope + ch0 + local) : 0.0F;
				q[j].bias = p.bias ? __ldg(p.bias + ch0 + local) : 0.0F;
			}
			const size_t stride4 = (size_t(p.c) * hw) >> 2;
			const size_t base4 = (((size_t(e0) * p.c + ch0) * hw) >> 2) + v;
			const float4 * x4 = reinterpret_cast<const float4 *>(p.x) + base4;
			const float4 * r4 = reinterpret_cast<const float4 *>(has_res ? p.res : p.x) + base4;
			float4 * y4 = reinterpret_cast<float4 *>(p.y) + base4;
			for (uint32_t e = e0; e < e1; e += U)
			{
				float4 xv[U], rv[U];
				#pragma unroll
				for (int u = 0; u < U; ++u)
				{
					rv[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					if (e + u < e1)
					{
						xv[u] = ld_stream(x4 + size_t(e + u - e0) * stride4);
						if (has_res)
							rv[u] = ld_stream(r4 + size_t(e + u - e0) * stride4);
					}
				}
				#pragma unroll
				for (int u = 0; u < U; ++u)
					if (e + u < e1)
					{
						float4 o;
						o.x = ew_element<A0, A1>(p, has_bn, has_res, q[0], xv[u].x, rv[u].x);
						o.y = ew_element<A0, A1>(p, has_bn, has_res, q[1], xv[u].y, rv[u].y);
						o.z = ew_element<A0, A1>(p, has_bn, has_res, q[2], xv[u].z, rv[u].z);
						o.w = ew_element<A0, A1>(p, has_bn, has_res, q[3], xv[u].w, rv[u].w);
						st_stream(y4 + size_t(e + u - e0) * stride4, o);
					}
			}
		}

		// false: the shape keeps the flat kernel
		bool plan_grouped(ewg_geom& g, int64_t n, int64_t c, int64_t hw)
		{
			if (hw % 4 == 0 || tune().no_grouped == 1 || n < 8 || n > 0x7fffffff || c > 0x7fffffff)
				return false;
			const int64_t unit = (hw % 2 == 0) ? 2 : 4;
			const int64_t vpu = unit * hw / 4;       // vectors of one unit of channels
			if (c % unit != 0 || vpu > kThreads)
				return false;
			int64_t group = unit * (kThreads / vpu);
			if (group > c)
				group = c;
			if (group * hw / 4 < 64)                 // CTAs of fewer than two warps: the flat kernel does better
				return false;
			g.n = (uint32_t)n;
			g.group = (uint32_t)group;
			g.groups = (uint32_t)div_up(c, group);
			g.threads = (uint32_t)(div_up(group * hw / 4, 32) * 32);
			const int64_t waves = tune().elementwise_group_waves > 0 ? tune().elementwise_group_waves : 2;
			int64_t split = div_up(int64_t(sm_count()) * 8 * waves, g.groups);
			if (split > n / 4) split = n / 4;
			if (split < 1) split = 1;
			g.entries_per_cta = (uint32_t)div_up(n, split);
			g.split = (uint32_t)div_up(n, g.entries_per_cta);
			g.d_hw = fastdiv((uint32_t)hw);
			return true;
		}

		cudaError_t launch_grouped(const ew_params& p, const ewg_geom& g, cudaStream_t s)
		{
			const int k0 = p.chain.n > 0 ? p.chain.a[0].kind : NNF_ACT_NONE;
			const int k1 = p.chain.n > 1 ? p.chain.a[1].kind : NNF_ACT_NONE;
			const unsigned grid = g.groups * g.split;
			const size_t smem = size_t(2) * g.group * sizeof(float);
#define NNF_EWG_CASE(A0, A1) bn_act_grouped_kernel<A0, A1><<<grid, g.threads, smem, s>>>(p, g)
			if (p.chain.n == 0)
				NNF_EWG_CASE(NNF_ACT_NONE, 0);
			else if (k0 == NNF_ACT_RELU && k1 == NNF_ACT_NONE)
				NNF_EWG_CASE(NNF_ACT_RELU, 0);
			else if (k0 == NNF_ACT_PRELU && k1 == NNF_ACT_ELU)
				NNF_EWG_CASE(NNF_ACT_PRELU, NNF_ACT_ELU);
			else
				NNF_EWG_CASE(-1, 0);
#undef NNF_EWG_CASE
			return cudaGetLastError();
		}

		// Grid: a whole number of resident waves (a grid somewhat larger than one wave would run a short second wave
		// with most SMs idle), never more than there are tiles. Measured on B200: CTAs that start at different times mix
		// their loads and stores, which a single wave moving in lockstep does not (2 GiB BN+TanH: 84 % of the copy
		// bandwidth with one wave, 94 % with 4, 102 % with 16, 104 % with 32); but every CTA fills the per-channel table
		// first, and below 64 tiles per resident CTA slot that cost shows (x[1024,256,14,14] BN+ReLU: 74 us with one wave,
		// 66 us with eight, 69 us with 32). So 32 waves for large tensors, eight otherwise.
		template <int MODE, int A0, int A1>
		int resident_grid(size_t smem, int64_t work)
		{
			// cached per kernel instantiation and shared-memory size (the size changes with the channel count)
			static int per_sm = 0;
			static size_t cached_smem = ~size_t(0);
			if (per_sm == 0 || cached_smem != smem)
			{
				int v = 0;
				if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, bn_act_kernel<MODE, A0, A1>, kThreads, smem) != cudaSuccess || v < 1)
				{
					cudaGetLastError();
					v = 4;
				}
				per_sm = v;
				cached_smem = smem;
			}
			const int forced = tune().elementwise_waves;   // grid size in units of one resident wave
			const int64_t wave = int64_t(sm_count()) * per_sm;
			const int waves = forced > 0 ? forced : (work >= 64 * wave ? 32 : 8);
			const int64_t cap = wave * waves;
			const int64_t g = work < cap ? work : cap;
			return g < 1 ? 1 : (int)g;
		}

		template <int MODE>
		cudaError_t launch_mode(const ew_params& p, int64_t work, size_t smem, cudaStream_t s)
		{
			const int k0 = p.chain.n > 0 ? p.chain.a[0].kind : NNF_ACT_NONE;
			const int k1 = p.chain.n > 1 ? p.chain.a[1].kind : NNF_ACT_NONE;
#define NNF_EW_CASE(A0, A1) bn_act_kernel<MODE, A0, A1><<<resident_grid<MODE, A0, A1>(smem, work), kThreads, smem, s>>>(p)
			if (k1 == NNF_ACT_NONE)
			{
				switch (k0)
				{
				case NNF_ACT_NONE: NNF_EW_CASE(NNF_ACT_NONE, 0); break;
				case NNF_ACT_RELU: NNF_EW_CASE(NNF_ACT_RELU, 0); break;
				case NNF_ACT_PRELU: NNF_EW_CASE(NNF_ACT_PRELU, 0); break;
				case NNF_ACT_ELU: NNF_EW_CASE(NNF_ACT_ELU, 0); break;
				case NNF_ACT_TANH: NNF_EW_CASE(NNF_ACT_TANH, 0); break;
				case NNF_ACT_SIGMOID: NNF_EW_CASE(NNF_ACT_SIGMOID, 0); break;
				default: NNF_EW_CASE(-1, 0); break;
				}
			}
			else if (k0 == NNF_ACT_PRELU && k1 == NNF_ACT_ELU)
				NNF_EW_CASE(NNF_ACT_PRELU, NNF_ACT_ELU);
			else
				NNF_EW_CASE(-1, 0);
#undef NNF_EW_CASE
			return cudaGetLastError();
		}
	}

	int run_elementwise(cudaStream_t s, float * y, const float * x, const float * res, float add_alpha,
		const bn_source& bn, const act_chain& chain, int64_t n, int64_t c, int64_t hw)
	{
		{
			const float * gamma = bn.gamma;
			const float * beta = bn.beta;
			const float * mean = bn.mean;
			const float * invsigma = bn.invsigma;
			const int64_t per_entry = c * hw;
			const int64_t total = n * per_entry;
			if (total == 0)
				return NNF_OK;
			bool need_channel = gamma != nullptr || bn.bias != nullptr;
			const float * slope = nullptr;
			for (int i = 0; i < chain.n; ++i)
				if (chain.a[i].kind == NNF_ACT_PRELU)
				{
					if (slope)
						return set_error(NNF_ERR_UNSUPPORTED, "at most one PReLU per fused chain");
					slope = chain.a[i].slope;
					need_channel = true;
				}

			// launches are split at entry boundaries when per-channel parameters are in play (so that
			// plane % C stays valid) and at multiples of 4 elements otherwise
			int64_t step;
			if (need_channel)
			{
				if (per_entry > kMaxElemsPerLaunch)
					return set_error(NNF_ERR_UNSUPPORTED, "one entry has %lld elements; at most %lld are supported per entry", (long long)per_entry, (long long)kMaxElemsPerLaunch);
				step = (kMaxElemsPerLaunch / per_entry) * per_entry;
			}
			else
				step = kMaxElemsPerLaunch & ~int64_t(3);

			for (int64_t off = 0; off < total; off += step)
			{
				const int64_t cnt = (total - off < step) ? (total - off) : step;
				ew_params p;
				p.y = y + off;
				p.x = x + off;
				p.res = res ? res + off : nullptr;
				p.gamma = gamma; p.beta = beta; p.mean = mean; p.invsigma = invsigma;
				p.sums = bn.sums; p.saved = (off == 0) ? bn.saved : nullptr; p.count_total = bn.count_total; p.eps = bn.eps;
				p.add_alpha = add_alpha;
				p.count = (uint32_t)cnt;
				p.c = (uint32_t)c;
				p.hw = fastdiv((uint32_t)hw);
				p.cdiv = fastdiv((uint32_t)c);
				p.slope = slope;
				p.bias = bn.bias;
				p.need_channel = need_channel ? 1 : 0;
				p.smem_params = (gamma && c <= kMaxSmemChannels) ? 1 : 0;
				if (bn.sums && !p.smem_params)
					return set_error(NNF_ERR_UNSUPPORTED, "training batch norm supports at most %d channels", kMaxSmemChannels);
				p.chain = chain;
				const size_t smem = p.smem_params ? size_t(2) * c * sizeof(float) : 0;
				const bool vec_ok = aligned16(p.y) && aligned16(p.x) && (!p.res || aligned16(p.res));
				const int mode = !vec_ok ? 2 : ((!need_channel || (hw % 4 == 0)) ? 0 : 1);
				const int64_t work = (mode == 2) ? div_up(cnt, kThreads) : div_up(cnt / 4 + 1, kThreads * kUnroll);
				cudaError_t e;
				ewg_geom gg;
				if (mode == 1 && plan_grouped(gg, cnt / per_entry, c, hw))
					e = launch_grouped(p, gg, s);
				else if (mode == 0)
					e = launch_mode<0>(p, work, smem, s);
				else if (mode == 1)
					e = launch_mode<1>(p, work, smem, s);
				else
					e = launch_mode<2>(p, work, smem, s);
				if (e != cudaSuccess)
					return set_error(NNF_ERR_CUDA, "bn_act_kernel launch failed: %s", cudaGetErrorString(e));
			}
			return NNF_OK;
		}
	}

	namespace
	{
		// ---- activation backward ---------------------------------------------------------------
		struct bw_params
		{
			float * dx;
			const float * dy;
			const float * t;      // layer input (ReLU, PReLU) or layer output (ELU, TanH, Sigmoid)
			const float * slope;
			float p0, p1;
			uint32_t count;
			uint32_t c;
			fastdiv hw;
			fastdiv cdiv;
			int add;
		};

		template <int KIND, int MODE>
		__global__ void __launch_bounds__(kThreads) act_bwd_kernel(const bw_params p)
		{
			auto channel_of = [&](uint32_t e) -> uint32_t {
				const uint32_t plane = p.hw.div(e);
				return plane - p.cdiv.div(plane) * p.c;
			};
			if (MODE == 2)
			{
				const uint32_t stride = gridDim.x * kThreads;
				for (uint32_t e = blockIdx.x * kThreads + threadIdx.x; e < p.count; e += stride)
				{
					const float a = (KIND == NNF_ACT_PRELU) ? __ldg(p.slope + channel_of(e)) : 0.0F;
					const float g = act_bwd<KIND>(p.dy[e], p.t[e], p.p0, p.p1, a);
					p.dx[e] = p.add ? __fadd_rn(p.dx[e], g) : g;
				}
				return;
			}
			const uint32_t nvec = p.count >> 2;
			const float4 * dy4 = reinterpret_cast<const float4 *>(p.dy);
			const float4 * t4 = reinterpret_cast<const float4 *>(p.t);
			float4 * dx4 = reinterpret_cast<float4 *>(p.dx);
			const uint32_t tile = kThreads * kUnroll;
			const uint32_t ntiles = (nvec + tile - 1) / tile;
			for (uint32_t tl = blockIdx.x; tl < ntiles; tl += gridDim.x)
			{
				const uint32_t v0 = tl * tile + threadIdx.x;
				float4 gv[kUnroll], tv[kUnroll], ov[kUnroll];
				#pragma unroll
				for (int j = 0; j < kUnroll; ++j)
				{
					const uint32_t v = v0 + j * kThreads;
					if (v < nvec)
					{
						gv[j] = ld_stream(dy4 + v);
						tv[j] = ld_stream(t4 + v);
						if (p.add)
							ov[j] = ld_stream(dx4 + v);
					}
				}
				#pragma unroll
				for (int j = 0; j < kUnroll; ++j)
				{
					const uint32_t v = v0 + j * kThreads;
					if (v < nvec)
					{
						const uint32_t e = v << 2;
						const float g[4] = {gv[j].x, gv[j].y, gv[j].z, gv[j].w};
						const float t[4] = {tv[j].x, tv[j].y, tv[j].z, tv[j].w};
						float o[4] = {0.0F, 0.0F, 0.0F, 0.0F};
						if (p.add)
						{
							o[0] = ov[j].x; o[1] = ov[j].y; o[2] = ov[j].z; o[3] = ov[j].w;
						}
						float a = 0.0F, a_next = 0.0F;
						uint32_t left = 4;   // elements of the vector that belong to its first channel
						if (KIND == NNF_ACT_PRELU && MODE == 0)
							a = __ldg(p.slope + channel_of(e));
						if (KIND == NNF_ACT_PRELU && MODE == 1 && p.hw.d >= 4)
						{
							// planes of at least four elements that are not whole vectors: a vector touches at most two channels
							const uint32_t plane = p.hw.div(e);
							const uint32_t channel = plane - p.cdiv.div(plane) * p.c;
							left = (plane + 1) * p.hw.d - e;
							a = __ldg(p.slope + channel);
							a_next = __ldg(p.slope + (channel + 1 == p.c ? 0 : channel + 1));
						}
						#pragma unroll
						for (int k = 0; k < 4; ++k)
						{
							float ak = a;
							if (KIND == NNF_ACT_PRELU && MODE == 1)
								ak = p.hw.d >= 4 ? (uint32_t(k) >= left ? a_next : a) : __ldg(p.slope + channel_of(e + k));
							const float r = act_bwd<KIND>(g[k], t[k], p.p0, p.p1, ak);
							o[k] = p.add ? __fadd_rn(o[k], r) : r;
						}
						st_stream(dx4 + v, make_float4(o[0], o[1], o[2], o[3]));
					}
				}
			}
			const uint32_t tail0 = nvec << 2;
			if (blockIdx.x == 0 && tail0 + threadIdx.x < p.count)
			{
				const uint32_t e = tail0 + threadIdx.x;
				const float a = (KIND == NNF_ACT_PRELU) ? __ldg(p.slope + channel_of(e)) : 0.0F;
				const float g = act_bwd<KIND>(p.dy[e], p.t[e], p.p0, p.p1, a);
				p.dx[e] = p.add ? __fadd_rn(p.dx[e], g) : g;
			}
		}

		template <int KIND>
		cudaError_t launch_bwd(const bw_params& p, int mode, int grid, cudaStream_t s)
		{
			if (mode == 0)
				act_bwd_kernel<KIND, 0><<<grid, kThreads, 0, s>>>(p);
			else if (mode == 1)
				act_bwd_kernel<KIND, 1><<<grid, kThreads, 0, s>>>(p);
			else
				act_bwd_kernel<KIND, 2><<<grid, kThreads, 0, s>>>(p);
			return cudaGetLastError();
		}

		// ---- n-ary add -------------------------------------------------------------------------
		struct add_params
		{
			float * y;
			const float * in[NNF_MAX_ADD_INPUTS];
			int k;
			float alpha;
			uint32_t count;
		};

		template <int MODE>
		__global__ void __launch_bounds__(kThreads) add_kernel(const add_params p)
		{
			if (MODE == 2)
			{
				const uint32_t stride = gridDim.x * kThreads;
				for (uint32_t e = blockIdx.x * kThreads + threadIdx.x; e < p.count; e += stride)
				{
					float sum = 0.0F;
					for (int j = 0; j < p.k; ++j)
						sum = __fadd_rn(sum, p.in[j][e]);
					p.y[e] = __fmul_rn(sum, p.alpha);
				}
				return;
			}
			const uint32_t nvec = p.count >> 2;
			float4 * y4 = reinterpret_cast<float4 *>(p.y);
			const uint32_t stride = gridDim.x * kThreads;
			for (uint32_t v = blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride)
			{
				float4 sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
				#pragma unroll
				for (int j = 0; j < NNF_MAX_ADD_INPUTS; ++j)
				{
					if (j < p.k)
					{
						const float4 a = ld_stream(reinterpret_cast<const float4 *>(p.in[j]) + v);
						sum.x = __fadd_rn(sum.x, a.x); sum.y = __fadd_rn(sum.y, a.y);
						sum.z = __fadd_rn(sum.z, a.z); sum.w = __fadd_rn(sum.w, a.w);
					}
				}
				st_stream(y4 + v, make_float4(__fmul_rn(sum.x, p.alpha), __fmul_rn(sum.y, p.alpha), __fmul_rn(sum.z, p.alpha), __fmul_rn(sum.w, p.alpha)));
			}
			const uint32_t tail0 = nvec << 2;
			if (blockIdx.x == 0 && tail0 + threadIdx.x < p.count)
			{
				const uint32_t e = tail0 + threadIdx.x;
				float sum = 0.0F;
				for (int j = 0; j < p.k; ++j)
					sum = __fadd_rn(sum, p.in[j][e]);
				p.y[e] = __fmul_rn(sum, p.alpha);
			}
		}

		// dx (+)= dy * alpha
		template <int MODE>
		__global__ void __launch_bounds__(kThreads) scale_kernel(float * dx, const float * dy, float alpha, uint32_t count, int add)
		{
			if (MODE == 2)
			{
				const uint32_t stride = gridDim.x * kThreads;
				for (uint32_t e = blockIdx.x * kThreads + threadIdx.x; e < count; e += stride)
				{
					const float g = __fmul_rn(dy[e], alpha);
					dx[e] = add ? __fadd_rn(dx[e], g) : g;
				}
				return;
			}
			const uint32_t nvec = count >> 2;
			float4 * dx4 = reinterpret_cast<float4 *>(dx);
			const float4 * dy4 = reinterpret_cast<const float4 *>(dy);
			const uint32_t stride = gridDim.x * kThreads;
			for (uint32_t v = blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride)
			{
				const float4 g = ld_stream(dy4 + v);
				float4 o = make_float4(__fmul_rn(g.x, alpha), __fmul_rn(g.y, alpha), __fmul_rn(g.z, alpha), __fmul_rn(g.w, alpha));
				if (add)
				{
					const float4 d = ld_stream(dx4 + v);
					o = make_float4(__fadd_rn(d.x, o.x), __fadd_rn(d.y, o.y), __fadd_rn(d.z, o.z), __fadd_rn(d.w, o.w));
				}
				st_stream(dx4 + v, o);
			}
			const uint32_t tail0 = nvec << 2;
			if (blockIdx.x == 0 && tail0 + threadIdx.x < count)
			{
				const uint32_t e = tail0 + threadIdx.x;
				const float g = __fmul_rn(dy[e], alpha);
				dx[e] = add ? __fadd_rn(dx[e], g) : g;
			}
		}

		int grid_for(int64_t cnt, int per_thread_vec)
		{
			int64_t work = div_up(cnt / 4 + 1, int64_t(kThreads) * per_thread_vec);
			const int64_t cap = int64_t(sm_count()) * kCtasPerSm;
			if (work > cap)
				work = cap;
			return work < 1 ? 1 : (int)work;
		}
	}

	int make_chain(act_chain& out, const nnf_act * acts, int n_acts, bool allow_prelu)
	{
		out.n = 0;
		for (int i = 0; i < NNF_MAX_ACTS; ++i)
		{
			out.a[i].kind = NNF_ACT_NONE;
			out.a[i].p0 = out.a[i].p1 = out.a[i].p0b = out.a[i].p1b = 0.0F;
			out.a[i].slope = nullptr;
		}
		if (n_acts < 0 || n_acts > NNF_MAX_ACTS)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "n_acts = %d, expected 0..%d", n_acts, NNF_MAX_ACTS);
		if (n_acts > 0 && !acts)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "acts is null with n_acts = %d", n_acts);
		for (int i = 0; i < n_acts; ++i)
		{
			act_param a;
			a.kind = acts[i].kind;
			a.p0 = acts[i].p0;
			a.p1 = acts[i].p1;
			a.slope = acts[i].slope;
			a.p0b = a.p1b = 0.0F;
			switch (a.kind)
			{
			case NNF_ACT_NONE:
				continue;
			case NNF_ACT_RELU:
			case NNF_ACT_ELU:
			case NNF_ACT_SIGMOID:
				break;
			case NNF_ACT_PRELU:
				if (!allow_prelu)
					return set_error(NNF_ERR_INVALID_ARGUMENT, "PReLU needs channel extents and cannot be used here");
				if (!a.slope)
					return set_error(NNF_ERR_INVALID_ARGUMENT, "PReLU activation without a slope buffer");
				break;
			case NNF_ACT_TANH:
				// device code wants steepness*2 (hyperbolic_tangent_layer_tester_plain.cpp:44)
				a.p1 = acts[i].p1 * 2.0F;
				break;
			default:
				return set_error(NNF_ERR_INVALID_ARGUMENT, "unknown activation kind %d", a.kind);
			}
			out.a[out.n++] = a;
		}
		return NNF_OK;
	}
}

using namespace nnf;

extern "C" int nnf_bn_infer_act(nnf_stream_t stream, float * y, const float * x,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	const float * residual, float add_alpha, const nnf_act * acts, int n_acts,
	int64_t n, int64_t c, int64_t hw)
{
	if (n < 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_infer_act: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (n == 0)
		return NNF_OK;
	if (!y || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_infer_act: null tensor pointer");
	if (gamma && (!beta || !mean || !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_infer_act: gamma given but beta/mean/invsigma missing");
	if (c > 0x7fffffff || hw > 0x7fffffff)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_infer_act: extent too large");
	act_chain chain;
	int st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	bn_source bn = {};
	bn.gamma = gamma; bn.beta = beta; bn.mean = mean; bn.invsigma = invsigma;
	return run_elementwise((cudaStream_t)stream, y, x, residual, add_alpha, bn, chain, n, c, hw);
}

extern "C" int nnf_bias_bn_infer_act(nnf_stream_t stream, float * y, const float * x, const float * bias,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	const float * residual, float add_alpha, const nnf_act * acts, int n_acts,
	int64_t n, int64_t c, int64_t hw)
{
	if (n < 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bias_bn_infer_act: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (n == 0)
		return NNF_OK;
	if (!y || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bias_bn_infer_act: null tensor pointer");
	if (gamma && (!beta || !mean || !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bias_bn_infer_act: gamma given but beta/mean/invsigma missing");
	if (c > 0x7fffffff || hw > 0x7fffffff)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bias_bn_infer_act: extent too large");
	act_chain chain;
	int st = make_chain(chain, acts, n_acts, true);
	if (st != NNF_OK)
		return st;
	bn_source bn = {};
	bn.gamma = gamma; bn.beta = beta; bn.mean = mean; bn.invsigma = invsigma;
	bn.bias = bias;
	return run_elementwise((cudaStream_t)stream, y, x, residual, add_alpha, bn, chain, n, c, hw);
}

extern "C" int nnf_act_fwd(nnf_stream_t stream, float * y, const float * x, const nnf_act * act, int64_t n, int64_t c, int64_t hw)
{
	return nnf_bn_infer_act(stream, y, x, nullptr, nullptr, nullptr, nullptr, nullptr, 1.0F, act, act ? 1 : 0, n, c, hw);
}

extern "C" int nnf_act_bwd(nnf_stream_t stream, float * dx, const float * dy, const float * neurons, const nnf_act * act,
	int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	if (n < 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_act_bwd: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (n == 0)
		return NNF_OK;
	if (!dx || !dy || !act)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_act_bwd: null pointer");
	if (act->kind != NNF_ACT_NONE && !neurons)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_act_bwd: the neurons buffer (input for ReLU/PReLU, output otherwise) is required");
	if (act->kind == NNF_ACT_PRELU && !act->slope)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_act_bwd: PReLU without a slope buffer");
	const int64_t per_entry = c * hw;
	const int64_t total = n * per_entry;
	const bool need_channel = act->kind == NNF_ACT_PRELU;
	if (need_channel && per_entry > kMaxElemsPerLaunch)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_act_bwd: entry too large");
	const int64_t step = need_channel ? (kMaxElemsPerLaunch / per_entry) * per_entry : (kMaxElemsPerLaunch & ~int64_t(3));
	for (int64_t off = 0; off < total; off += step)
	{
		const int64_t cnt = (total - off < step) ? (total - off) : step;
		bw_params p;
		p.dx = dx + off;
		p.dy = dy + off;
		p.t = neurons ? neurons + off : dy + off;
		p.slope = act->slope;
		p.p0 = act->p0;
		p.p1 = act->p1;
		if (act->kind == NNF_ACT_TANH)
		{
			// hyperbolic_tangent_layer_updater_plain.cpp:87-88
			p.p0 = 1.0F / act->p0;
			p.p1 = act->p1 * act->p0;
		}
		p.count = (uint32_t)cnt;
		p.c = (uint32_t)c;
		p.hw = fastdiv((uint32_t)hw);
		p.cdiv = fastdiv((uint32_t)c);
		p.add = add_to_destination ? 1 : 0;
		const bool vec_ok = aligned16(p.dx) && aligned16(p.dy) && aligned16(p.t);
		const int mode = !vec_ok ? 2 : ((!need_channel || (hw % 4 == 0)) ? 0 : 1);
		const int grid = (mode == 2) ? grid_for(cnt * 4, 1) : grid_for(cnt, kUnroll);
		cudaError_t e;
		switch (act->kind)
		{
		case NNF_ACT_NONE: e = launch_bwd<NNF_ACT_NONE>(p, mode, grid, (cudaStream_t)stream); break;
		case NNF_ACT_RELU: e = launch_bwd<NNF_ACT_RELU>(p, mode, grid, (cudaStream_t)stream); break;
		case NNF_ACT_PRELU: e = launch_bwd<NNF_ACT_PRELU>(p, mode, grid, (cudaStream_t)stream); break;
		case NNF_ACT_ELU: e = launch_bwd<NNF_ACT_ELU>(p, mode, grid, (cudaStream_t)stream); break;
		case NNF_ACT_TANH: e = launch_bwd<NNF_ACT_TANH>(p, mode, grid, (cudaStream_t)stream); break;
		case NNF_ACT_SIGMOID: e = launch_bwd<NNF_ACT_SIGMOID>(p, mode, grid, (cudaStream_t)stream); break;
		default: return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_act_bwd: unknown activation kind %d", act->kind);
		}
		if (e != cudaSuccess)
			return set_error(NNF_ERR_CUDA, "act_bwd_kernel launch failed: %s", cudaGetErrorString(e));
	}
	return NNF_OK;
}

extern "C" int nnf_add_fwd(nnf_stream_t stream, float * y, const float * const * inputs, int input_count, float alpha, int64_t count)
{
	if (count < 0 || input_count < 1 || input_count > NNF_MAX_ADD_INPUTS)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_add_fwd: count=%lld input_count=%d (1..%d)", (long long)count, input_count, NNF_MAX_ADD_INPUTS);
	if (count == 0)
		return NNF_OK;
	if (!y || !inputs)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_add_fwd: null pointer");
	for (int j = 0; j < input_count; ++j)
		if (!inputs[j])
			return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_add_fwd: input %d is null", j);
	const int64_t step = kMaxElemsPerLaunch & ~int64_t(3);
	for (int64_t off = 0; off < count; off += step)
	{
		const int64_t cnt = (count - off < step) ? (count - off) : step;
		add_params p;
		p.y = y + off;
		bool vec_ok = aligned16(p.y);
		for (int j = 0; j < NNF_MAX_ADD_INPUTS; ++j)
		{
			p.in[j] = j < input_count ? inputs[j] + off : nullptr;
			vec_ok = vec_ok && (j >= input_count || aligned16(p.in[j]));
		}
		p.k = input_count;
		p.alpha = alpha;
		p.count = (uint32_t)cnt;
		if (vec_ok)
			add_kernel<0><<<grid_for(cnt, 1), kThreads, 0, (cudaStream_t)stream>>>(p);
		else
			add_kernel<2><<<grid_for(cnt * 4, 1), kThreads, 0, (cudaStream_t)stream>>>(p);
		cudaError_t e = cudaGetLastError();
		if (e != cudaSuccess)
			return set_error(NNF_ERR_CUDA, "add_kernel launch failed: %s", cudaGetErrorString(e));
	}
	return NNF_OK;
}

extern "C" int nnf_add_bwd(nnf_stream_t stream, float * dx, const float * dy, float alpha, int64_t count, int add_to_destination)
{
	if (count < 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_add_bwd: count=%lld", (long long)count);
	if (count == 0)
		return NNF_OK;
	if (!dx || !dy)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_add_bwd: null pointer");
	if (!add_to_destination && dx == dy && alpha == 1.0F)
		return NNF_OK; // add_layer_updater_plain.cpp:98: nothing to do in place with unit scale
	const int64_t step = kMaxElemsPerLaunch & ~int64_t(3);
	for (int64_t off = 0; off < count; off += step)
	{
		const int64_t cnt = (count - off < step) ? (count - off) : step;
		if (aligned16(dx + off) && aligned16(dy + off))
			scale_kernel<0><<<grid_for(cnt, 1), kThreads, 0, (cudaStream_t)stream>>>(dx + off, dy + off, alpha, (uint32_t)cnt, add_to_destination ? 1 : 0);
		else
			scale_kernel<2><<<grid_for(cnt * 4, 1), kThreads, 0, (cudaStream_t)stream>>>(dx + off, dy + off, alpha, (uint32_t)cnt, add_to_destination ? 1 : 0);
		cudaError_t e = cudaGetLastError();
		if (e != cudaSuccess)
			return set_error(NNF_ERR_CUDA, "scale_kernel launch failed: %s", cudaGetErrorString(e));
	}
	return NNF_OK;
}
