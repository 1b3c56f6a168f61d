// The weight-update side of the per-channel layers:
//  * nnf_apply_gradient: the optimiser step of nnforge/cuda/util_cuda.cu:337-596 (plain SGD, vanilla and Nesterov
//    momentum, ADAM) for MANY weight chunks in one launch. The reference launches one kernel per chunk
//    (backward_propagation_cuda.cpp:2008-2096): four for a batch-norm layer (gamma, beta, mean, inverse sigma), one
//    for a PReLU layer, each a few KB, so a network's per-channel weights cost hundreds of launches per step. Here
//    a table of chunks travels by value in the kernel parameters and every CTA looks up the chunk it serves.
//  * nnf_bn_calibrate_*: the statistics collection behind toolset::update_bn_weights (nnforge/toolset.cpp:1562-1630)
//    as a GPU reduction: per feature map the count / mean / M2 / min / max of the batch-norm output computed with
//    gamma 1 and beta 0, merged across batches in double, and the rewrite of mean and inverse sigma from them.
#include "nnf_common.cuh"

#include <math.h>

namespace nnf
{
	namespace
	{
		constexpr int kOptThreads = 256;
		constexpr int kOptPerThread = 4;
		constexpr uint32_t kOptPerCta = kOptThreads * kOptPerThread;
		constexpr int kOptMaxParts = 48;            // chunks per launch; sized to keep the parameter block under 4 KB
		constexpr uint32_t kOptMaxPartElems = 1u << 30;

		struct opt_part
		{
			float * data;
			float * gradient;
			float * prev_upd;
			float * prev_upd2;
			double * update_accum;
			float learning_rate;
			float weight_decay;
			uint32_t count;
			uint32_t first_cta;
		};

		struct opt_params
		{
			opt_part part[kOptMaxParts];
			int n_parts;
			float normalizer;
			float momentum, momentum_plus1;      // vanilla / Nesterov; ADAM: momentum = beta1
			float beta2, one_minus_beta1, one_minus_beta2;
			float inv1, inv2, epsilon;           // ADAM bias corrections 1 / (1 - beta^t)
		};

		__device__ __forceinline__ double warp_sum(double v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v += __shfl_xor_sync(0xffffffffu, v, o);
			return v;
		}

		// TYPE: nnf_momentum_type. Every product and sum is rounded on its own, in the order the plain backend
		// writes them (nnforge/plain/backward_propagation_plain.cpp:826-985).
		template <int TYPE>
		__global__ void __launch_bounds__(kOptThreads) apply_gradient_kernel(const __grid_constant__ opt_params p)
		{
			__shared__ double s_red[kOptThreads / 32];
			int k = 0;
			while (k + 1 < p.n_parts && blockIdx.x >= p.part[k + 1].first_cta)
				++k;
			const opt_part& part = p.part[k];
			const uint32_t base = (blockIdx.x - part.first_cta) * kOptPerCta;
			double acc = 0.0;
			#pragma unroll
			for (int u = 0; u < kOptPerThread; ++u)
			{
				const uint32_t i = base + u * kOptThreads + threadIdx.x;
				if (i >= part.count)
					break;
				const float w = part.data[i];
				const float gr = part.gradient[i];
				const float total = __fsub_rn(__fmul_rn(gr, p.normalizer), __fmul_rn(w, part.weight_decay));
				float upd;
				if (TYPE == NNF_MOMENTUM_NONE)
					upd = __fmul_rn(part.learning_rate, total);
				else if (TYPE == NNF_MOMENTUM_VANILLA)
				{
					upd = __fadd_rn(__fmul_rn(part.prev_upd[i], p.momentum), __fmul_rn(part.learning_rate, total));
					part.prev_upd[i] = upd;
				}
				else if (TYPE == NNF_MOMENTUM_NESTEROV)
				{
					const float prev = part.prev_upd[i];
					const float fresh = __fadd_rn(__fmul_rn(prev, p.momentum), __fmul_rn(part.learning_rate, total));
					upd = __fsub_rn(__fmul_rn(p.momentum_plus1, fresh), __fmul_rn(p.momentum, prev));
					part.prev_upd[i] = fresh;
				}
				else
				{
					const float m1 = __fadd_rn(__fmul_rn(p.momentum, part.prev_upd[i]), __fmul_rn(p.one_minus_beta1, total));
					const float m2 = __fadd_rn(__fmul_rn(p.beta2, part.prev_upd2[i]), __fmul_rn(__fmul_rn(p.one_minus_beta2, total), total));
					const float u1 = __fmul_rn(m1, p.inv1), u2 = __fmul_rn(m2, p.inv2);
					upd = __fdiv_rn(__fmul_rn(part.learning_rate, u1), __fadd_rn(__fsqrt_rn(u2), p.epsilon));
					part.prev_upd[i] = m1;
					part.prev_upd2[i] = m2;
				}
				part.data[i] = __fadd_rn(w, upd);
				part.gradient[i] = 0.0F;
				acc += double(fabsf(upd));
			}
			if (part.update_accum)   // uniform per CTA
			{
				acc = warp_sum(acc);
				if ((threadIdx.x & 31) == 0)
					s_red[threadIdx.x >> 5] = acc;
				__syncthreads();
				if (threadIdx.x == 0)
				{
					double t = 0.0;
					for (int i = 0; i < kOptThreads / 32; ++i)
						t += s_red[i];
					// a chunk of up to 1024 weights has one CTA, so its sum has a fixed order; larger chunks add
					// their CTAs' sums in arrival order
					atomicAdd(part.update_accum, t);
				}
			}
		}

		// ---- batch-norm calibration --------------------------------------------------------------------
		constexpr int kCalThreads = 256;
		constexpr int kCalLoads = 4;
		constexpr int kCalMaxSplit = 64;
		constexpr int kCalPartials = 4;   // sum, sum of squares, min, max

		struct cal_params
		{
			const float * x;
			const float * mean;
			const float * invsigma;
			double * partial;          // [c][split][kCalPartials]
			double * acc;              // [5][c]: count, mean, M2, min, max
			uint32_t n, c, hw, split, entries_per_cta;
			fastdiv d_per_plane;
			int vec;
		};

		struct cal_acc
		{
			double s = 0.0, q = 0.0;
			float lo = 3.402823466e+38F, hi = -3.402823466e+38F;

			__device__ __forceinline__ void take(float x, float mult, float add)
			{
				// the inference batch norm with gamma 1, beta 0 (nnforge/plain/batch_norm_layer_tester_plain.cpp:66-84):
				// the value whose statistics the reference collects
				const float y = __fadd_rn(__fmul_rn(x, mult), add);
				const double yd = double(y);
				s += yd;
				q += yd * yd;
				lo = fminf(lo, y);
				hi = fmaxf(hi, y);
			}
		};

		__global__ void __launch_bounds__(kCalThreads) bn_calibrate_stats_kernel(const cal_params p)
		{
			__shared__ double s_red[kCalThreads / 32][kCalPartials];
			const uint32_t ch = blockIdx.x / p.split;
			const uint32_t sp = blockIdx.x - ch * p.split;
			const uint32_t e0 = sp * p.entries_per_cta;
			const uint32_t e1 = min(e0 + p.entries_per_cta, p.n);
			const float mult = p.invsigma[ch];                        // gamma * invsigma with gamma = 1
			const float add = __fsub_rn(0.0F, __fmul_rn(mult, p.mean[ch]));   // beta - mult * mean with beta = 0
			cal_acc a;
			if (e0 < e1)
			{
				const uint32_t per_plane = p.vec ? (p.hw >> 2) : p.hw;
				const uint32_t total = (e1 - e0) * per_plane;
				const size_t entry_stride = size_t(p.c) * p.hw;
				const float * base = p.x + (size_t(e0) * p.c + ch) * p.hw;
				for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kCalThreads * kCalLoads)
				{
					if (p.vec)
					{
						float4 v[kCalLoads];
						#pragma unroll
						for (int u = 0; u < kCalLoads; ++u)
						{
							const uint32_t i = i0 + u * kCalThreads;
							if (i < total)
							{
								const uint32_t lp = p.d_per_plane.div(i);
								v[u] = __ldcs(reinterpret_cast<const float4 *>(base + lp * entry_stride) + (i - lp * per_plane));
							}
						}
						#pragma unroll
						for (int u = 0; u < kCalLoads; ++u)
							if (i0 + u * kCalThreads < total)
							{
								a.take(v[u].x, mult, add);
								a.take(v[u].y, mult, add);
								a.take(v[u].z, mult, add);
								a.take(v[u].w, mult, add);
							}
					}
					else
					{
						float v[kCalLoads];
						#pragma unroll
						for (int u = 0; u < kCalLoads; ++u)
						{
							const uint32_t i = i0 + u * kCalThreads;
							if (i < total)
							{
								const uint32_t lp = p.d_per_plane.div(i);
								v[u] = __ldcs(base + lp * entry_stride + (i - lp * per_plane));
							}
						}
						#pragma unroll
						for (int u = 0; u < kCalLoads; ++u)
							if (i0 + u * kCalThreads < total)
								a.take(v[u], mult, add);
					}
				}
			}
			double s = warp_sum(a.s), q = warp_sum(a.q);
			float lo = a.lo, hi = a.hi;
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
			{
				lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
				hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
			}
			const int w = threadIdx.x >> 5;
			if ((threadIdx.x & 31) == 0)
			{
				s_red[w][0] = s;
				s_red[w][1] = q;
				s_red[w][2] = double(lo);
				s_red[w][3] = double(hi);
			}
			__syncthreads();
			if (threadIdx.x == 0)
			{
				for (int i = 1; i < kCalThreads / 32; ++i)
				{
					s_red[0][0] += s_red[i][0];
					s_red[0][1] += s_red[i][1];
					s_red[0][2] = fmin(s_red[0][2], s_red[i][2]);
					s_red[0][3] = fmax(s_red[0][3], s_red[i][3]);
				}
				double * out = p.partial + (size_t(ch) * p.split + sp) * kCalPartials;
				for (int k = 0; k < kCalPartials; ++k)
					out[k] = s_red[0][k];
			}
		}

		// Folds one batch's partials per feature map, in slice order, and merges the batch into the running
		// count / mean / M2 with the pairwise update of Chan et al., so that the result does not depend on how the data
		// set was cut into batches beyond double rounding.
		__global__ void bn_calibrate_merge_kernel(const cal_params p)
		{
			const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
			if (ch >= p.c)
				return;
			double s = 0.0, q = 0.0, lo = 3.402823466e+38, hi = -3.402823466e+38;
			for (uint32_t sp = 0; sp < p.split; ++sp)
			{
				const double * in = p.partial + (size_t(ch) * p.split + sp) * kCalPartials;
				s += in[0];
				q += in[1];
				lo = fmin(lo, in[2]);
				hi = fmax(hi, in[3]);
			}
			const double nb = double(p.n) * double(p.hw);
			const double mean_b = s / nb;
			const double m2_b = fmax(q - s * mean_b, 0.0);
			double * acc = p.acc;
			const double na = acc[ch];
			if (na == 0.0)
			{
				acc[ch] = nb;
				acc[p.c + ch] = mean_b;
				acc[2 * size_t(p.c) + ch] = m2_b;
				acc[3 * size_t(p.c) + ch] = lo;
				acc[4 * size_t(p.c) + ch] = hi;
			}
			else
			{
				const double nt = na + nb;
				const double delta = mean_b - acc[p.c + ch];
				acc[ch] = nt;
				acc[p.c + ch] += delta * (nb / nt);
				acc[2 * size_t(p.c) + ch] += m2_b + delta * delta * (na * nb / nt);
				acc[3 * size_t(p.c) + ch] = fmin(acc[3 * size_t(p.c) + ch], lo);
				acc[4 * size_t(p.c) + ch] = fmax(acc[4 * size_t(p.c) + ch], hi);
			}
		}

		// stat_data_bunch_writer::get_stat (nnforge/stat_data_bunch_writer.cpp:83-111) and the rewrite of the running
		// statistics (nnforge/toolset.cpp:1613-1620)
		__global__ void bn_calibrate_finish_kernel(float * mean, float * invsigma, float * stats, const double * acc, uint32_t c)
		{
			const uint32_t ch = blockIdx.x * blockDim.x + threadIdx.x;
			if (ch >= c)
				return;
			const float average = float(acc[c + ch]);
			const float std_dev = __fsqrt_rn(float(acc[2 * size_t(c) + ch] / acc[ch]));
			if (stats)
			{
				stats[ch] = float(acc[3 * size_t(c) + ch]);
				stats[c + ch] = float(acc[4 * size_t(c) + ch]);
				stats[2 * size_t(c) + ch] = average;
				stats[3 * size_t(c) + ch] = std_dev;
			}
			if (mean)
			{
				const float old_mean = mean[ch], old_invsigma = invsigma[ch];
				invsigma[ch] = __fdiv_rn(old_invsigma, std_dev);
				mean[ch] = __fadd_rn(old_mean, __fdiv_rn(average, old_invsigma));
			}
		}
	}
}

using namespace nnf;

extern "C" int nnf_apply_gradient(nnf_stream_t stream, const nnf_opt_part * parts, int n_parts, int momentum_type, float momentum,
	float momentum2, float normalizer, unsigned int iteration_id)
{
	if (n_parts < 0 || (n_parts > 0 && !parts))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_apply_gradient: bad chunk list");
	if (momentum_type < NNF_MOMENTUM_NONE || momentum_type > NNF_MOMENTUM_ADAM)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_apply_gradient: unknown momentum type %d", momentum_type);
	if (momentum_type == NNF_MOMENTUM_ADAM && iteration_id == 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_apply_gradient: ADAM counts iterations from 1");
	opt_params p;
	p.normalizer = normalizer;
	p.momentum = momentum;
	p.momentum_plus1 = momentum + 1.0F;
	p.beta2 = momentum2;
	p.one_minus_beta1 = 1.0F - momentum;
	p.one_minus_beta2 = 1.0F - momentum2;
	p.inv1 = p.inv2 = 0.0F;
	p.epsilon = 1.0e-8F;
	if (momentum_type == NNF_MOMENTUM_ADAM)
	{
		// nnforge/cuda/util_cuda.cu: the bias corrections are evaluated on the host in fp32
		p.inv1 = 1.0F / (1.0F - powf(momentum, float(iteration_id)));
		p.inv2 = 1.0F / (1.0F - powf(momentum2, float(iteration_id)));
	}
	for (int k = 0; k < n_parts; ++k)
	{
		const nnf_opt_part& s = parts[k];
		if (s.elem_count < 0 || (s.elem_count > 0 && (!s.data || !s.gradient)))
			return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_apply_gradient: chunk %d has no data or gradient", k);
		if (s.elem_count > 0 && momentum_type != NNF_MOMENTUM_NONE && !s.prev_upd)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_apply_gradient: chunk %d needs the previous update", k);
		if (s.elem_count > 0 && momentum_type == NNF_MOMENTUM_ADAM && !s.prev_upd2)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_apply_gradient: chunk %d needs the second moment", k);
	}
	cudaStream_t cs = (cudaStream_t)stream;
	auto flush = [&](uint32_t ctas) -> int
	{
		if (p.n_parts == 0)
			return NNF_OK;
		switch (momentum_type)
		{
		case NNF_MOMENTUM_NONE: apply_gradient_kernel<NNF_MOMENTUM_NONE><<<ctas, kOptThreads, 0, cs>>>(p); break;
		case NNF_MOMENTUM_VANILLA: apply_gradient_kernel<NNF_MOMENTUM_VANILLA><<<ctas, kOptThreads, 0, cs>>>(p); break;
		case NNF_MOMENTUM_NESTEROV: apply_gradient_kernel<NNF_MOMENTUM_NESTEROV><<<ctas, kOptThreads, 0, cs>>>(p); break;
		default: apply_gradient_kernel<NNF_MOMENTUM_ADAM><<<ctas, kOptThreads, 0, cs>>>(p); break;
		}
		p.n_parts = 0;
		return check_launch("apply_gradient_kernel");
	};
	p.n_parts = 0;
	uint32_t ctas = 0;
	for (int k = 0; k < n_parts; ++k)
	{
		const nnf_opt_part& s = parts[k];
		// chunks beyond 2^30 weights are served as several table entries that share the accumulator
		for (int64_t off = 0; off < s.elem_count; off += kOptMaxPartElems)
		{
			const uint32_t count = uint32_t(s.elem_count - off < int64_t(kOptMaxPartElems) ? s.elem_count - off : int64_t(kOptMaxPartElems));
			const uint32_t need = (count + kOptPerCta - 1) / kOptPerCta;
			if (p.n_parts == kOptMaxParts || ctas + need > 0x7fffffffu)
			{
				const int rc = flush(ctas);
				if (rc != NNF_OK)
					return rc;
				ctas = 0;
			}
			opt_part& d = p.part[p.n_parts++];
			d.data = s.data + off;
			d.gradient = s.gradient + off;
			d.prev_upd = s.prev_upd ? s.prev_upd + off : nullptr;
			d.prev_upd2 = s.prev_upd2 ? s.prev_upd2 + off : nullptr;
			d.update_accum = s.update_accum;
			d.learning_rate = s.learning_rate;
			d.weight_decay = s.weight_decay;
			d.count = count;
			d.first_cta = ctas;
			ctas += need;
		}
	}
	return flush(ctas);
}

extern "C" size_t nnf_bn_calibrate_workspace_bytes(int64_t c)
{
	return c > 0 ? size_t(c) * kCalMaxSplit * kCalPartials * sizeof(double) : 0;
}

extern "C" size_t nnf_bn_calibrate_accumulator_bytes(int64_t c)
{
	return c > 0 ? size_t(c) * 5 * sizeof(double) : 0;
}

extern "C" int nnf_bn_calibrate_accumulate(nnf_stream_t stream, void * accumulator, const float * x, const float * mean, const float * invsigma,
	int64_t n, int64_t c, int64_t hw, void * workspace, size_t workspace_bytes)
{
	if (!accumulator || !x || !mean || !invsigma || n <= 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_calibrate_accumulate: null pointer or empty shape");
	if (!workspace || workspace_bytes < nnf_bn_calibrate_workspace_bytes(c))
		return set_error(NNF_ERR_WORKSPACE, "nnf_bn_calibrate_accumulate: workspace of %zu bytes needed", nnf_bn_calibrate_workspace_bytes(c));
	if (n >= (int64_t(1) << 31) || c >= (int64_t(1) << 25) || hw >= (int64_t(1) << 31))
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_calibrate_accumulate: extent too large");
	cal_params p;
	p.x = x;
	p.mean = mean;
	p.invsigma = invsigma;
	p.partial = static_cast<double *>(workspace);
	p.acc = static_cast<double *>(accumulator);
	p.n = uint32_t(n);
	p.c = uint32_t(c);
	p.hw = uint32_t(hw);
	p.vec = (hw % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
	int64_t split = (int64_t(sm_count()) * 8 + c - 1) / c;
	split = split < 1 ? 1 : split;
	split = split > kCalMaxSplit ? kCalMaxSplit : split;
	split = split > n ? n : split;
	int64_t per = (n + split - 1) / split;
	if (per * hw >= (int64_t(1) << 31))
	{
		// one CTA's slice must stay 32-bit indexable: use every slice the workspace allows
		split = n < kCalMaxSplit ? n : kCalMaxSplit;
		per = (n + split - 1) / split;
		if (per * hw >= (int64_t(1) << 31))
			return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_calibrate_accumulate: %lld entries of %lld values per feature map are too many for one call",
				(long long)n, (long long)hw);
	}
	split = (n + per - 1) / per;
	p.split = uint32_t(split);
	p.entries_per_cta = uint32_t(per);
	p.d_per_plane = fastdiv(p.vec ? p.hw >> 2 : p.hw);
	cudaStream_t cs = (cudaStream_t)stream;
	bn_calibrate_stats_kernel<<<uint32_t(c * split), kCalThreads, 0, cs>>>(p);
	int rc = check_launch("bn_calibrate_stats_kernel");
	if (rc != NNF_OK)
		return rc;
	bn_calibrate_merge_kernel<<<uint32_t((c + 127) / 128), 128, 0, cs>>>(p);
	return check_launch("bn_calibrate_merge_kernel");
}

extern "C" int nnf_bn_calibrate_finish(nnf_stream_t stream, float * mean, float * invsigma, float * stats, const void * accumulator, int64_t c)
{
	if (!accumulator || c <= 0 || (!mean != !invsigma) || (!mean && !stats))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_calibrate_finish: null pointer or empty shape");
	bn_calibrate_finish_kernel<<<uint32_t((c + 127) / 128), 128, 0, (cudaStream_t)stream>>>(mean, invsigma, stats,
		static_cast<const double *>(accumulator), uint32_t(c));
	return check_launch("bn_calibrate_finish_kernel");
}
