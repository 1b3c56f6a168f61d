/*
 * CPU restatement of nnForge's plain (CPU) backend for the batch-norm / activation / add /
 * softmax / max-subsampling path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the parity checker and the timed CPU baseline; the product
 * library never links, loads or calls it. Every function names the reference lines it follows
 * (paths relative to the reference project root). Expression order, accumulator seeds and scan
 * order are kept exactly as in those lines because the parity bar is bit-exactness for ReLU and
 * max-pool results. Build with -O2 -ffp-contract=off and without -ffast-math (oracle/build_oracle.py).
 *
 * Pinning: each function below that has a reference counterpart is compared bit-for-bit against the
 * reference's own sources compiled in place (oracle/build_ref.py -> oracle/_ref) by
 * tests/test_oracle_vs_reference.py wherever a reference checkout is present, and against the
 * golden vectors under tests/golden/ (generated from that reference build) everywhere else.
 * Training-mode batch norm (orc_bn_train_*) has NO reference CPU implementation - the reference
 * calls cuDNN there - so its parity is UNPINNED by reference code; it restates the documented
 * spatial batch-norm formulas and is cross-checked against a double-precision twin and against
 * PyTorch's CPU batch_norm in the tests. The optimiser step (orc_apply_gradient) and the three-line rewrite of the
 * running statistics (orc_bn_recalibrate) follow reference files that need Boost to compile
 * (plain/backward_propagation_plain.cpp, toolset.cpp): their parity is UNPINNED too; the optimiser is checked bit for bit
 * against an independent numpy float32 statement of the same formulas (tests/test_oracle_golden.py). The statistics the
 * recalibration consumes (orc_feature_map_stats_*) ARE pinned, to the reference's stat_data_bunch_writer.cpp.
 *
 * Layout everywhere: planar fp32, offset = ((n*C + c)*H + y)*W + x.
 * With -fopenmp the outer loops run in parallel exactly where the reference has its
 * "#pragma omp parallel for"; results do not depend on the thread count except where stated.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#define ORC_PAR _Pragma("omp parallel for schedule(guided)")
#else
#define ORC_PAR
#endif

typedef int64_t i64;

int orc_max_threads(void)
{
#ifdef _OPENMP
	return omp_get_max_threads();
#else
	return 1;
#endif
}

/* The OpenMP build only: how many threads the loops below use (a launcher may have set OMP_NUM_THREADS=1 for the
 * process; the timed CPU baseline is meant to use every core it is allowed). */
void orc_set_threads(int n)
{
#ifdef _OPENMP
	if (n > 0)
		omp_set_num_threads(n);
#else
	(void)n;
#endif
}

/* ---- batch norm, inference: nnforge/plain/batch_norm_layer_tester_plain.cpp:30-75 ------------
 * mult = gamma*invsigma; add = beta - mult*mean (both rounded to fp32, per (entry, channel));
 * y = x*mult + add with a separately rounded product (no fused multiply-add). */
void orc_bn_infer(float * y, const float * x, const float * gamma, const float * beta, const float * mean,
	const float * invsigma, i64 n, i64 c, i64 hw)
{
	const i64 total = n * c;
	i64 w;
	ORC_PAR
	for (w = 0; w < total; ++w)
	{
		const i64 ch = w % c;
		const float mult = gamma[ch] * invsigma[ch];
		const float add = beta[ch] - mult * mean[ch];
		const float * in = x + w * hw;
		float * out = y + w * hw;
		i64 i;
		for (i = 0; i < hw; ++i)
			out[i] = in[i] * mult + add;
	}
}

/* ---- ReLU: nnforge/plain/rectified_linear_layer_tester_plain.cpp:50-55 -------------------------
 * Negative inputs are multiplied by the slope, so slope 0 produces -0.0f. */
void orc_relu_fwd(float * y, const float * x, float slope, i64 count)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		const float v = x[i];
		y[i] = v >= 0.0F ? v : v * slope;
	}
}

/* nnforge/plain/rectified_linear_layer_updater_plain.cpp:62-107: gate on the INPUT value. */
void orc_relu_bwd(float * dx, const float * dy, const float * x, float slope, i64 count, int add_to_destination)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		const float g = (x[i] >= 0.0F) ? dy[i] : dy[i] * slope;
		if (add_to_destination)
			dx[i] += g;
		else
			dx[i] = g;
	}
}

/* ---- PReLU: nnforge/plain/parametric_rectified_linear_layer_tester_plain.cpp:51-70 ------------- */
void orc_prelu_fwd(float * y, const float * x, const float * slope, i64 n, i64 c, i64 hw)
{
	const i64 total = n * c;
	i64 w;
	ORC_PAR
	for (w = 0; w < total; ++w)
	{
		const float a = slope[w % c];
		const float * in = x + w * hw;
		float * out = y + w * hw;
		i64 i;
		for (i = 0; i < hw; ++i)
			out[i] = in[i] * (in[i] >= 0.0F ? 1.0F : a);
	}
}

/* nnforge/plain/parametric_rectified_linear_layer_updater_plain.cpp:74-135 */
void orc_prelu_bwd_data(float * dx, const float * dy, const float * x, const float * slope, i64 n, i64 c, i64 hw,
	int add_to_destination)
{
	const i64 total = n * c;
	i64 w;
	ORC_PAR
	for (w = 0; w < total; ++w)
	{
		const float a = slope[w % c];
		i64 i;
		for (i = 0; i < hw; ++i)
		{
			const i64 k = w * hw + i;
			const float g = dy[k] * (x[k] >= 0.0F ? 1.0F : a);
			if (add_to_destination)
				dx[k] += g;
			else
				dx[k] = g;
		}
	}
}

/* nnforge/plain/parametric_rectified_linear_layer_updater_plain.cpp:137-190: per channel, an fp32
 * sum over the pixels of one entry, then an fp32 sum of those over entries, ADDED to the gradient. */
void orc_prelu_bwd_weights(float * dslope, const float * dy, const float * x, i64 n, i64 c, i64 hw)
{
	i64 ch;
	ORC_PAR
	for (ch = 0; ch < c; ++ch)
	{
		float sum = 0.0F;
		i64 e;
		for (e = 0; e < n; ++e)
		{
			const i64 base = (e * c + ch) * hw;
			float local_sum = 0.0F;
			i64 i;
			for (i = 0; i < hw; ++i)
				local_sum += dy[base + i] * (x[base + i] >= 0.0F ? 0.0F : x[base + i]);
			sum += local_sum;
		}
		dslope[ch] += sum;
	}
}

/* ---- ELU (alpha fixed at 1): nnforge/plain/exponential_linear_layer_tester_plain.cpp:48-53 ----- */
void orc_elu_fwd(float * y, const float * x, i64 count)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
		y[i] = x[i] >= 0.0F ? x[i] : (expf(x[i]) - 1.0F);
}

/* nnforge/plain/exponential_linear_layer_updater_plain.cpp:59-103: derivative from the OUTPUT. */
void orc_elu_bwd(float * dx, const float * dy, const float * y, i64 count, int add_to_destination)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		const float der = (y[i] >= 0) ? 1.0F : (y[i] + 1.0F);
		if (add_to_destination)
			dx[i] += dy[i] * der;
		else
			dx[i] = dy[i] * der;
	}
}

/* ---- TanH: nnforge/plain/hyperbolic_tangent_layer_tester_plain.cpp:47-58 ---------------------- */
void orc_tanh_fwd(float * y, const float * x, float scale, float steepness, i64 count)
{
	const float steepness2 = steepness * 2.0F;
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		const float e = expf(x[i] * steepness2);
		y[i] = (e - 1.0F) / (e + 1.0F) * scale;
	}
}

/* nnforge/plain/hyperbolic_tangent_layer_updater_plain.cpp:62-112 */
void orc_tanh_bwd(float * dx, const float * dy, const float * y, float scale, float steepness, i64 count, int add_to_destination)
{
	const float scale_reverse = 1.0F / scale;
	const float steepness3 = steepness * scale;
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		const float nv = y[i] * scale_reverse;
		const float der = steepness3 * (1.0F - (nv * nv));
		if (add_to_destination)
			dx[i] += dy[i] * der;
		else
			dx[i] = dy[i] * der;
	}
}

/* ---- Sigmoid: nnforge/plain/sigmoid_layer_tester_plain.cpp:47-53 ------------------------------ */
void orc_sigmoid_fwd(float * y, const float * x, i64 count)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
		y[i] = 1.0F / (expf(-x[i]) + 1.0F);
}

/* nnforge/plain/sigmoid_layer_updater_plain.cpp:59-103 */
void orc_sigmoid_bwd(float * dx, const float * dy, const float * y, i64 count, int add_to_destination)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		const float der = y[i] * (1.0F - y[i]);
		if (add_to_destination)
			dx[i] += dy[i] * der;
		else
			dx[i] = dy[i] * der;
	}
}

/* ---- Add: nnforge/plain/add_layer_tester_plain.cpp:53-61 ---------------------------------------
 * The accumulator starts at +0.0f and the scale is applied to the finished sum. */
void orc_add_fwd(float * y, const float * const * inputs, int input_count, float alpha, i64 count)
{
	i64 i;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		float sum = 0.0F;
		int j;
		for (j = 0; j < input_count; ++j)
			sum += inputs[j][i];
		y[i] = sum * alpha;
	}
}

/* nnforge/plain/add_layer_updater_plain.cpp:66-109 (in place with alpha == 1 is a no-op there). */
void orc_add_bwd(float * dx, const float * dy, float alpha, i64 count, int add_to_destination)
{
	i64 i;
	if (!add_to_destination && dx == dy && alpha == 1.0F)
		return;
	ORC_PAR
	for (i = 0; i < count; ++i)
	{
		if (add_to_destination)
			dx[i] += dy[i] * alpha;
		else
			dx[i] = dy[i] * alpha;
	}
}

/* ---- Softmax over channels: nnforge/plain/softmax_layer_tester_plain.cpp:65-88 -----------------
 * max seeded with -1.0e37f, ascending-c fp32 sum, multiply by the rounded reciprocal. */
void orc_softmax_fwd(float * y, const float * x, i64 n, i64 c, i64 hw)
{
	const i64 total = n * hw;
	i64 w;
	ORC_PAR
	for (w = 0; w < total; ++w)
	{
		const i64 e = w / hw;
		const i64 p = w - e * hw;
		const float * in = x + e * c * hw + p;
		float * out = y + e * c * hw + p;
		float max_val = -1.0e+37F;
		float sum = 0.0F;
		float mult;
		i64 f;
		for (f = 0; f < c; ++f)
		{
			const float v = in[f * hw];
			max_val = (max_val < v) ? v : max_val; /* std::max(max_val, v) */
		}
		for (f = 0; f < c; ++f)
		{
			const float v = expf(in[f * hw] - max_val);
			sum += v;
			out[f * hw] = v;
		}
		mult = 1.0F / sum;
		for (f = 0; f < c; ++f)
			out[f * hw] *= mult;
	}
}

/* nnforge/plain/softmax_layer_updater_plain.cpp:100-166 */
void orc_softmax_bwd(float * dx, const float * dy, const float * y, i64 n, i64 c, i64 hw, int add_to_destination)
{
	const i64 total = n * hw;
	i64 w;
	ORC_PAR
	for (w = 0; w < total; ++w)
	{
		const i64 e = w / hw;
		const i64 p = w - e * hw;
		const i64 base = e * c * hw + p;
		float sum = 0.0F;
		i64 f;
		for (f = 0; f < c; ++f)
			sum += dy[base + f * hw] * y[base + f * hw];
		for (f = 0; f < c; ++f)
		{
			const float g = y[base + f * hw] * (dy[base + f * hw] - sum);
			if (add_to_destination)
				dx[base + f * hw] += g;
			else
				dx[base + f * hw] = g;
		}
	}
}

/* ---- Max subsampling ---------------------------------------------------------------------------
 * Output extent: nnforge/max_subsampling_layer.cpp:125-133. */
i64 orc_maxpool_out_size(i64 in_size, i64 window, i64 stride, int round_up)
{
	return (in_size + stride - window + (round_up ? window - 1 : 0)) / stride;
}

/* Forward with argmax: nnforge/plain/max_subsampling_layer_updater_plain.cpp:118-168.
 * The window is scanned x-fastest (offset table of :99-115), the first element always seeds the
 * result and a later one replaces it only on a strict ">" ("<" for is_min). argmax holds the
 * ABSOLUTE input element offset as unsigned int, or may be NULL (tester variant,
 * nnforge/plain/max_subsampling_layer_tester_plain.cpp:170-288).
 * round_up is refused by the plain backend (:60-62); here it clips the window to the input, which
 * is what the reference CUDA kernel does (nnforge/cuda/max_subsampling_layer_updater_cuda.cuh:108-150). */
void orc_maxpool_fwd(float * y, uint32_t * argmax, const float * x, i64 n, i64 c, i64 h, i64 w,
	i64 win_w, i64 win_h, i64 stride_w, i64 stride_h, int round_up_w, int round_up_h, int is_min)
{
	const i64 ow = orc_maxpool_out_size(w, win_w, stride_w, round_up_w);
	const i64 oh = orc_maxpool_out_size(h, win_h, stride_h, round_up_h);
	const i64 planes = n * c;
	i64 pl;
	ORC_PAR
	for (pl = 0; pl < planes; ++pl)
	{
		const float * in = x + pl * h * w;
		i64 oy, ox;
		for (oy = 0; oy < oh; ++oy)
			for (ox = 0; ox < ow; ++ox)
			{
				float best = is_min ? 1.0e37F : -1.0e37F;
				i64 best_index = 0;
				int first = 1;
				i64 ky, kx;
				for (ky = 0; ky < win_h; ++ky)
				{
					const i64 iy = oy * stride_h + ky;
					if (iy >= h)
						break;
					for (kx = 0; kx < win_w; ++kx)
					{
						const i64 ix = ox * stride_w + kx;
						float v;
						if (ix >= w)
							break;
						v = in[iy * w + ix];
						if (first || ((v > best) && !is_min) || ((v < best) && is_min))
						{
							best = v;
							best_index = pl * h * w + iy * w + ix;
							first = 0;
						}
					}
				}
				y[(pl * oh + oy) * ow + ox] = best;
				if (argmax)
					argmax[(pl * oh + oy) * ow + ox] = (uint32_t)best_index;
			}
	}
}

/* Backward: nnforge/plain/max_subsampling_layer_updater_plain.cpp:173-231, in the only form that is
 * well defined for overlapping windows: destination zero-filled unless accumulating, then
 * "dx[argmax[o]] += dy[o]" serially in ascending output index o. (The reference's non-accumulating
 * branch assigns instead of adding and both branches run under an OpenMP loop, which loses or races
 * contributions when windows overlap; its CUDA twin zero-fills and adds atomically.) Always serial. */
void orc_maxpool_bwd(float * dx, const float * dy, const uint32_t * argmax, i64 in_count, i64 out_count, int add_to_destination)
{
	i64 o;
	if (!add_to_destination)
		memset(dx, 0, (size_t)in_count * sizeof(float));
	for (o = 0; o < out_count; ++o)
		dx[argmax[o]] += dy[o];
}

/* ---- Batch norm, training mode (NO reference CPU code; parity unpinned) ------------------------
 * Replaces the two cuDNN calls at nnforge/cuda/batch_norm_layer_updater_cuda.cu:89-106 and :145-164.
 * Documented spatial batch norm: mean = sum(x)/m, biased var = sum((x-mean)^2)/m,
 * invstd = 1/sqrt(var+eps). The normalisation is then applied in the inference form of
 * nnforge/plain/batch_norm_layer_tester_plain.cpp:60-72 (mult = gamma*invstd, add = beta - mult*mean,
 * y = x*mult + add) so that the sign of y - which gates the following PReLU/ELU - is decided by one
 * expression in forward and backward.
 *
 * Statistics are accumulated in double here (the "exact" twin); orc_bn_train_stats_f32 is the fp32
 * form using the only per-channel reduction order the reference owns (per-entry inner sum, then
 * across entries: nnforge/plain/parametric_rectified_linear_layer_updater_plain.cpp:166-188).
 * count_total lets a caller pass statistics summed over several shards (synchronised batch norm). */
void orc_bn_train_sums(double * sum, double * sumsq, const float * x, i64 n, i64 c, i64 hw)
{
	i64 ch;
	ORC_PAR
	for (ch = 0; ch < c; ++ch)
	{
		double s = 0.0, q = 0.0;
		i64 e, i;
		for (e = 0; e < n; ++e)
		{
			const float * in = x + (e * c + ch) * hw;
			for (i = 0; i < hw; ++i)
			{
				s += in[i];
				q += (double)in[i] * in[i];
			}
		}
		sum[ch] = s;
		sumsq[ch] = q;
	}
}

void orc_bn_train_sums_f32(float * sum, float * sumsq, const float * x, i64 n, i64 c, i64 hw)
{
	i64 ch;
	ORC_PAR
	for (ch = 0; ch < c; ++ch)
	{
		float s = 0.0F, q = 0.0F;
		i64 e, i;
		for (e = 0; e < n; ++e)
		{
			const float * in = x + (e * c + ch) * hw;
			float ls = 0.0F, lq = 0.0F;
			for (i = 0; i < hw; ++i)
			{
				ls += in[i];
				lq += in[i] * in[i];
			}
			s += ls;
			q += lq;
		}
		sum[ch] = s;
		sumsq[ch] = q;
	}
}

/* mean/invstd from (already global) sums over count_total elements per channel; written as
 * saved[0:c] = mean, saved[c:2c] = invstd, the layout of the reference's temporary_fixed_buffer
 * (nnforge/cuda/batch_norm_layer_updater_cuda.cu:105-106). */
void orc_bn_train_finalize(float * saved, const double * sum, const double * sumsq, i64 c, double count_total, float eps)
{
	i64 ch;
	for (ch = 0; ch < c; ++ch)
	{
		const double mean = sum[ch] / count_total;
		double var = sumsq[ch] / count_total - mean * mean;
		if (var < 0.0)
			var = 0.0;
		saved[ch] = (float)mean;
		saved[c + ch] = (float)(1.0 / sqrt(var + (double)eps));
	}
}

/* y = x*mult + add with the saved statistics. */
void orc_bn_train_apply(float * y, const float * x, const float * gamma, const float * beta, const float * saved, i64 n, i64 c, i64 hw)
{
	orc_bn_infer(y, x, gamma, beta, saved, saved + c, n, c, hw);
}

/* Per-channel backward sums in double: dbeta = sum(du), dgamma = sum(du * xhat),
 * xhat = (x - mean)*invstd evaluated in fp32. */
void orc_bn_train_bwd_sums(double * dbeta, double * dgamma, const float * du, const float * x, const float * saved, i64 n, i64 c, i64 hw)
{
	i64 ch;
	ORC_PAR
	for (ch = 0; ch < c; ++ch)
	{
		const float mean = saved[ch], invstd = saved[c + ch];
		double sb = 0.0, sg = 0.0;
		i64 e, i;
		for (e = 0; e < n; ++e)
		{
			const i64 base = (e * c + ch) * hw;
			for (i = 0; i < hw; ++i)
			{
				const float xhat = (x[base + i] - mean) * invstd;
				sb += du[base + i];
				sg += (double)du[base + i] * xhat;
			}
		}
		dbeta[ch] = sb;
		dgamma[ch] = sg;
	}
}

/* dx = gamma*invstd/m * (m*du - dbeta - xhat*dgamma), evaluated in double and rounded once;
 * accumulates when add_to_destination (cuDNN beta_data = 1 at :135). dbeta/dgamma are the global sums. */
void orc_bn_train_bwd_apply(float * dx, const float * du, const float * x, const float * gamma, const float * saved,
	const double * dbeta, const double * dgamma, i64 n, i64 c, i64 hw, double count_total, int add_to_destination)
{
	const i64 total = n * c;
	i64 w;
	ORC_PAR
	for (w = 0; w < total; ++w)
	{
		const i64 ch = w % c;
		const float mean = saved[ch], invstd = saved[c + ch];
		const double k = (double)gamma[ch] * invstd / count_total;
		i64 i;
		for (i = 0; i < hw; ++i)
		{
			const i64 idx = w * hw + i;
			const float xhat = (x[idx] - mean) * invstd;
			const float g = (float)(k * (count_total * du[idx] - dbeta[ch] - (double)xhat * dgamma[ch]));
			if (add_to_destination)
				dx[idx] += g;
			else
				dx[idx] = g;
		}
	}
}

/* Running-statistics pseudo-gradients: nnforge/cuda/batch_norm_layer_updater_cuda.cu:28-44,167-182.
 * grad_mean += entry_count*(batch_mean - mean), same for the inverse standard deviation. */
void orc_bn_train_running_grad(float * grad_mean, float * grad_invsigma, const float * saved, const float * mean, const float * invsigma,
	i64 c, float entry_count)
{
	i64 ch;
	for (ch = 0; ch < c; ++ch)
	{
		grad_mean[ch] += entry_count * (saved[ch] - mean[ch]);
		grad_invsigma[ch] += entry_count * (saved[c + ch] - invsigma[ch]);
	}
}

/* ---- Negative log likelihood over channels (the loss behind softmax) ------------------------------
 * nnforge/plain/negative_log_likelihood_layer_tester_plain.cpp:60-92 (the updater's forward is the same,
 * negative_log_likelihood_layer_updater_plain.cpp:60-92): per (entry, pixel)
 *   err = scale * mask * ( - sum over channels with actual > 0, ascending, of actual * logf(max(predicted, 1e-20)) )
 * accumulated as err -= term, then multiplied by the total scale; 0 when the total scale is 0. */
void orc_nll_fwd(float * err, const float * predicted, const float * actual, const float * mask, float scale, i64 n, i64 c, i64 hw)
{
	for (i64 e = 0; e < n; ++e)
		for (i64 p = 0; p < hw; ++p)
		{
			float total_scale = scale;
			if (mask)
				total_scale *= mask[e * hw + p];
			float v = 0.0F;
			if (total_scale != 0.0F)
			{
				for (i64 f = 0; f < c; ++f)
				{
					const float pr = predicted[(e * c + f) * hw + p];
					const float ac = actual[(e * c + f) * hw + p];
					if (ac > 0.0F)
						v -= ac * logf(pr < 1.0e-20F ? 1.0e-20F : pr); /* std::max(pr, 1e-20): a NaN prediction stays NaN */
				}
				v *= total_scale;
			}
			err[e * hw + p] = v;
		}
}

/* nnforge/plain/negative_log_likelihood_layer_updater_plain.cpp:131-157: gradient with respect to the predictions,
 *   g = (actual > 0 ? actual / max(predicted, 1e-20) : 0) * total_scale   (0 when the total scale is 0). */
void orc_nll_bwd(float * dpredicted, const float * predicted, const float * actual, const float * mask, float scale, i64 n, i64 c, i64 hw,
	int add_to_destination)
{
	for (i64 e = 0; e < n; ++e)
		for (i64 p = 0; p < hw; ++p)
		{
			float total_scale = scale;
			if (mask)
				total_scale *= mask[e * hw + p];
			for (i64 f = 0; f < c; ++f)
			{
				const i64 off = (e * c + f) * hw + p;
				float g = 0.0F;
				if (total_scale != 0.0F)
				{
					const float ac = actual[off], pr = predicted[off];
					if (ac > 0.0F)
						g = ac / (pr < 1.0e-20F ? 1.0e-20F : pr);
					g *= total_scale;
				}
				if (add_to_destination)
					dpredicted[off] += g;
				else
					dpredicted[off] = g;
			}
		}
}

/* ---- Cross entropy over channels (the loss behind sigmoid outputs) -----------------------------------
 * nnforge/plain/cross_entropy_layer_tester_plain.cpp:60-97 and cross_entropy_layer_updater_plain.cpp:62-99: per (entry, pixel)
 *   err = total_scale * sum over channels, ascending, of
 *           ( actual > 0 ? -actual * logf(max(predicted, 1e-20)) : 0 ) + ( actual < 1 ? -(1 - actual) * logf(max(1 - predicted, 1e-20)) : 0 )
 * accumulated as two separate err -= term steps per channel; 0 when the total scale is 0. The two files differ in the total scale
 * when a mask is given: the updater multiplies, total_scale = scale * mask (:71-73), the tester REPLACES the scale by the mask,
 * total_scale = mask (:72-74). mask_replaces_scale selects the tester's form. */
void orc_cross_entropy_fwd(float * err, const float * predicted, const float * actual, const float * mask, float scale, i64 n, i64 c, i64 hw,
	int mask_replaces_scale)
{
	for (i64 e = 0; e < n; ++e)
		for (i64 p = 0; p < hw; ++p)
		{
			float total_scale = scale;
			if (mask)
			{
				if (mask_replaces_scale)
					total_scale = mask[e * hw + p];
				else
					total_scale *= mask[e * hw + p];
			}
			float v = 0.0F;
			if (total_scale != 0.0F)
			{
				for (i64 f = 0; f < c; ++f)
				{
					const float pr = predicted[(e * c + f) * hw + p];
					const float ac = actual[(e * c + f) * hw + p];
					if (ac > 0.0F)
						v -= ac * logf(pr < 1.0e-20F ? 1.0e-20F : pr);
					if (ac < 1.0F)
					{
						const float q = 1.0F - pr;
						v -= (1.0F - ac) * logf(q < 1.0e-20F ? 1.0e-20F : q);
					}
				}
				v *= total_scale;
			}
			err[e * hw + p] = v;
		}
}

/* Gradient with respect to the predictions,
 *   g = ( (actual > 0 ? actual / max(predicted, 1e-20) : 0) - (actual < 1 ? (1 - actual) / max(1 - predicted, 1e-20) : 0) ) * scale * mask,
 * 0 when the total scale is 0. This is what cross_entropy_layer_updater_plain.cpp:146-166 computes - into a local `float gradient`
 * that shadows the one which is stored (:150 against :157), so the plain backend itself writes zeros; the CUDA backend stores the
 * value (nnforge/cuda/cross_entropy_layer_updater_cuda.cu:115-183). The one deviation from the plain backend on this path. */
void orc_cross_entropy_bwd(float * dpredicted, const float * predicted, const float * actual, const float * mask, float scale, i64 n, i64 c, i64 hw,
	int add_to_destination)
{
	for (i64 e = 0; e < n; ++e)
		for (i64 p = 0; p < hw; ++p)
		{
			float total_scale = scale;
			if (mask)
				total_scale *= mask[e * hw + p];
			for (i64 f = 0; f < c; ++f)
			{
				const i64 off = (e * c + f) * hw + p;
				float g = 0.0F;
				if (total_scale != 0.0F)
				{
					const float ac = actual[off], pr = predicted[off];
					if (ac > 0.0F)
						g = ac / (pr < 1.0e-20F ? 1.0e-20F : pr);
					if (ac < 1.0F)
					{
						const float q = 1.0F - pr;
						g -= (1.0F - ac) / (q < 1.0e-20F ? 1.0e-20F : q);
					}
					g *= total_scale;
				}
				if (add_to_destination)
					dpredicted[off] += g;
				else
					dpredicted[off] = g;
			}
		}
}

/* ---- Top-n accuracy over channels: nnforge/plain/accuracy_layer_tester_plain.cpp:64-110 -------------
 * Per (entry, pixel): the actual class is the first channel holding the largest target (strict >, seeded
 * -1e37); rank = number of channels whose prediction beats the prediction of the actual class (larger, or equal
 * with a smaller channel index). out[k] = (rank <= k ? mask : 0) for k < top_n, out[top_n] = mask; mask = 1
 * without a mask; a zero mask gives rank 0 without looking at the data. */
void orc_accuracy_fwd(float * out, const float * predicted, const float * actual, const float * mask, i64 top_n, i64 n, i64 c, i64 hw)
{
	for (i64 e = 0; e < n; ++e)
		for (i64 p = 0; p < hw; ++p)
		{
			const float m = mask ? mask[e * hw + p] : 1.0F;
			int sum = 0;
			if (m != 0.0F)
			{
				float max_val = -1.0e37F;
				i64 cls = -1;
				for (i64 f = 0; f < c; ++f)
				{
					const float a = actual[(e * c + f) * hw + p];
					if (a > max_val)
					{
						max_val = a;
						cls = f;
					}
				}
				/* cls stays -1 when no target exceeds the seed (all NaN): the reference then reads one plane before the
				 * entry; the restatement gives rank 0 for that degenerate input */
				if (cls >= 0)
				{
					max_val = predicted[(e * c + cls) * hw + p];
					for (i64 f = 0; f < c; ++f)
					{
						const float v = predicted[(e * c + f) * hw + p];
						if (v > max_val || (v == max_val && f < cls))
							++sum;
					}
				}
			}
			for (i64 k = 0; k < top_n; ++k)
				out[(e * (top_n + 1) + k) * hw + p] = sum <= k ? m : 0.0F;
			out[(e * (top_n + 1) + top_n) * hw + p] = m;
		}
}

/* ---- Average subsampling over the two spatial dimensions (windows do not overlap: stride = window) --------
 * nnforge/plain/average_subsampling_layer_tester_plain.cpp:120-135: the window is summed from +0 with x fastest, then
 * multiplied by mult (the effective alpha: 1 / window elements by default, average_subsampling_layer.cpp:287-301). */
void orc_avgpool_fwd(float * y, const float * x, i64 planes, i64 h, i64 w, i64 win_w, i64 win_h, float mult)
{
	const i64 oh = h / win_h, ow = w / win_w;
	for (i64 p = 0; p < planes; ++p)
		for (i64 oy = 0; oy < oh; ++oy)
			for (i64 ox = 0; ox < ow; ++ox)
			{
				float sum = 0.0F;
				for (i64 yy = 0; yy < win_h; ++yy)
					for (i64 xx = 0; xx < win_w; ++xx)
						sum += x[(p * h + oy * win_h + yy) * w + ox * win_w + xx];
				y[(p * oh + oy) * ow + ox] = sum * mult;
			}
}

/* nnforge/plain/average_subsampling_layer_updater_plain.cpp:270-285: every element of a window receives dy * mult. */
void orc_avgpool_bwd(float * dx, const float * dy, i64 planes, i64 h, i64 w, i64 win_w, i64 win_h, float mult, int add_to_destination)
{
	const i64 oh = h / win_h, ow = w / win_w;
	for (i64 p = 0; p < planes; ++p)
		for (i64 yy = 0; yy < h; ++yy)
			for (i64 xx = 0; xx < w; ++xx)
			{
				const float err = dy[(p * oh + yy / win_h) * ow + xx / win_w] * mult;
				float * o = dx + (p * h + yy) * w + xx;
				if (add_to_destination)
					*o += err;
				else
					*o = err;
			}
}

/* ---- optimiser step: nnforge/plain/backward_propagation_plain.cpp:826-985 (one weight chunk) ------------
 * momentum_type 0 none, 1 vanilla, 2 Nesterov, 3 ADAM (momentum = beta1, momentum2 = beta2, iteration counted from 1).
 * Returns the sum of |update| in double. weight_decay is the value that applies to this chunk, as in the CUDA
 * backend (nnforge/cuda/backward_propagation_cuda.cpp:2029-2031); the plain backend's ADAM branch uses the
 * ungated value and its no-momentum branch carries the |update| sum over from chunk to chunk.
 * This file of the reference needs Boost to compile, so this function is checked against the source by reading
 * only: parity unpinned. */
double orc_apply_gradient(float * data, float * gradient, float * prev_upd, float * prev_upd2, i64 count, int momentum_type,
	float learning_rate, float normalizer, float weight_decay, float momentum, float momentum2, unsigned int iteration_id)
{
	double accum = 0.0;
	const float mp1 = momentum + 1.0F;
	float inv1 = 0.0F, inv2 = 0.0F;
	const float epsilon = 1.0e-8F;
	i64 i;
	if (momentum_type == 3)
	{
		inv1 = 1.0F / (1.0F - powf(momentum, (float)iteration_id));
		inv2 = 1.0F / (1.0F - powf(momentum2, (float)iteration_id));
	}
	for (i = 0; i < count; ++i)
	{
		const float w = data[i], gr = gradient[i];
		float upd;
		if (momentum_type == 0)
			upd = learning_rate * (gr * normalizer - w * weight_decay);
		else if (momentum_type == 1)
		{
			upd = prev_upd[i] * momentum + learning_rate * (gr * normalizer - w * weight_decay);
			prev_upd[i] = upd;
		}
		else if (momentum_type == 2)
		{
			const float prev = prev_upd[i];
			const float fresh = prev * momentum + learning_rate * (gr * normalizer - w * weight_decay);
			upd = mp1 * fresh - momentum * prev;
			prev_upd[i] = fresh;
		}
		else
		{
			const float total = gr * normalizer - w * weight_decay;
			const float m1 = momentum * prev_upd[i] + (1.0F - momentum) * total;
			const float m2 = momentum2 * prev_upd2[i] + (1.0F - momentum2) * total * total;
			const float u1 = m1 * inv1, u2 = m2 * inv2;
			upd = learning_rate * u1 / (sqrtf(u2) + epsilon);
			prev_upd[i] = m1;
			prev_upd2[i] = m2;
		}
		accum += (double)fabsf(upd);
		data[i] = w + upd;
		gradient[i] = 0.0F;
	}
	return accum;
}

/* ---- per-feature-map statistics: nnforge/stat_data_bunch_writer.cpp:44-111 -------------------------------
 * state[c][3] = {n, mean, m2} (double) and minmax[c][2] carry over between calls (one call per batch of entries);
 * value by value update of Welford's single-pass algorithm, as the reference does per entry. */
void orc_feature_map_stats_update(double * state, float * minmax, const float * y, i64 n, i64 c, i64 hw)
{
	i64 e, ch, i;
	for (e = 0; e < n; ++e)
		for (ch = 0; ch < c; ++ch)
		{
			double * st = state + ch * 3;
			const float * in = y + (e * c + ch) * hw;
			for (i = 0; i < hw; ++i)
			{
				const float val = in[i];
				double val_d, delta, delta2;
				if (val < minmax[ch * 2]) minmax[ch * 2] = val;
				if (val > minmax[ch * 2 + 1]) minmax[ch * 2 + 1] = val;
				st[0] += 1.0;
				val_d = (double)val;
				delta = val_d - st[1];
				st[1] += delta / st[0];
				delta2 = val_d - st[1];
				st[2] += delta * delta2;
			}
		}
}

/* stats[4][c] = {min, max, average, std_dev}: stat_data_bunch_writer::get_stat, nnforge/stat_data_bunch_writer.cpp:83-111 */
void orc_feature_map_stats_get(float * stats, const double * state, const float * minmax, i64 c)
{
	i64 ch;
	for (ch = 0; ch < c; ++ch)
	{
		stats[ch] = minmax[ch * 2];
		stats[c + ch] = minmax[ch * 2 + 1];
		stats[2 * c + ch] = (float)state[ch * 3 + 1];
		stats[3 * c + ch] = sqrtf((float)(state[ch * 3 + 2] / state[ch * 3]));
	}
}

/* toolset::update_bn_weights, nnforge/toolset.cpp:1613-1620: the running statistics rewritten from the statistics of the
 * layer's output under gamma 1, beta 0. (toolset.cpp needs Boost to compile: checked against the source by reading.) */
void orc_bn_recalibrate(float * mean, float * invsigma, const float * stats, i64 c)
{
	i64 ch;
	for (ch = 0; ch < c; ++ch)
	{
		const float old_mean = mean[ch], old_invsigma = invsigma[ch];
		invsigma[ch] = old_invsigma / stats[3 * c + ch];
		mean[ch] = old_mean + stats[2 * c + ch] / old_invsigma;
	}
}
