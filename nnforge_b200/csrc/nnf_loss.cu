// The loss side of channel softmax: negative log likelihood (nnforge/plain/negative_log_likelihood_layer_*_plain.cpp,
// nnforge/cuda/negative_log_likelihood_layer_*_cuda.cu), stand-alone and fused with the softmax in front of it, and
// the top-n accuracy layer (end of the file).
//
//   forward : err[n][pixel]  = total_scale * ( - sum over channels with target > 0 of target * logf(max(p, 1e-20)) )
//   backward: dp[n][f][pixel] = (target > 0 ? target / max(p, 1e-20) : 0) * total_scale
//   total_scale = scale * mask[n][pixel] (mask optional); a total scale of 0 gives 0.
// Fused with softmax the probabilities never make the extra trips through HBM:
//   forward : logits, targets (, mask) -> p, err            12 B/element instead of 8 + 8 (+ tiny)
//   backward: p, targets (, mask)      -> dlogits           12 B/element instead of 12 + 12
// with exactly the operations of the two layers run one after the other (softmax as in nnf_softmax.cu, then the
// loss on the rounded probabilities; backward: the loss gradient g, then dlogit = p * (g - sum_f g_f p_f)).
//
// Two access patterns, as for softmax: H*W == 1 (classifier rows): a warp per row, the row in registers as
// float4 when C % 4 == 0 and C <= 1024, shuffle reductions; H*W > 1 (per-pixel): a thread per pixel, channels
// strided by H*W (coalesced across the warp), the column in registers when C <= 32, sums in ascending channel
// order like the plain backend. Other channel counts take the same kernels without the register copy: the row or
// column is read again (from L1/L2) by each pass.
#include "nnf_common.cuh"

namespace nnf
{
	namespace
	{
		constexpr float kLossMaxSeed = -1.0e+37F;   // softmax_layer_tester_plain.cpp:69
		constexpr float kLossFloor = 1.0e-20F;      // negative_log_likelihood_layer_tester_plain.cpp:85

		__device__ __forceinline__ float loss_ref_max(float a, float b) { return (a < b) ? b : a; } // std::max(a, b)

		__device__ __forceinline__ float loss_warp_max(float v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
			return v;
		}

		__device__ __forceinline__ float loss_warp_sum(float v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
			return v;
		}

		// one term of the loss and of its gradient
		__device__ __forceinline__ float nll_term(float p, float t)
		{
			// __logf (lg2.approx * ln 2): absolute error 2^-21.4 on [0.5, 2], 3 ulp elsewhere - inside the 1e-5 tolerance,
			// and cheap enough to run on every element: with one-hot targets nearly every warp has a lane with a
			// positive target in every channel, so a branch around a full logf would be taken by everybody
			return t > 0.0F ? __fmul_rn(t, __logf(loss_ref_max(p, kLossFloor))) : 0.0F;
		}

		__device__ __forceinline__ float nll_grad(float p, float t, float total_scale)
		{
			float g = 0.0F;
			if (total_scale != 0.0F)
			{
				if (t > 0.0F)
					g = __fdiv_rn(t, loss_ref_max(p, kLossFloor));
				g = __fmul_rn(g, total_scale);
			}
			return g;
		}

		struct loss_params
		{
			float * out;            // p (fused forward), dlogits (fused backward), dp (stand-alone backward); unused for stand-alone forward
			float * err;            // forward: [n][pixel]
			const float * in;       // logits (fused forward) or p
			const float * targets;
			const float * mask;     // [n][pixel] or null
			float scale;
			int c;
			int add;
			int64_t rows;           // H*W == 1: entries; else pixels of this launch
			uint32_t hw;
			fastdiv hwdiv;
		};

		enum { kFusedFwd = 0, kFusedBwd = 1, kLossFwd = 2, kLossBwd = 3, kCeFwd = 4, kCeBwd = 5 };

		// cross entropy (nnforge/plain/cross_entropy_layer_tester_plain.cpp:79-92): two terms per element, each subtracted on its own
		__device__ __forceinline__ float ce_accumulate(float e, float p, float t)
		{
			if (t > 0.0F)
				e = __fsub_rn(e, __fmul_rn(t, __logf(loss_ref_max(p, kLossFloor))));
			if (t < 1.0F)
				e = __fsub_rn(e, __fmul_rn(__fsub_rn(1.0F, t), __logf(loss_ref_max(__fsub_rn(1.0F, p), kLossFloor))));
			return e;
		}

		// the gradient cross_entropy_layer_updater_plain.cpp:146-166 computes (and, through a shadowed variable, fails to store;
		// the CUDA backend stores it, cross_entropy_layer_updater_cuda.cu:115-183)
		__device__ __forceinline__ float ce_grad(float p, float t, float total_scale)
		{
			float g = 0.0F;
			if (total_scale != 0.0F)
			{
				if (t > 0.0F)
					g = __fdiv_rn(t, loss_ref_max(p, kLossFloor));
				if (t < 1.0F)
					g = __fsub_rn(g, __fdiv_rn(__fsub_rn(1.0F, t), loss_ref_max(__fsub_rn(1.0F, p), kLossFloor)));
				g = __fmul_rn(g, total_scale);
			}
			return g;
		}

		template <int MODE>
		__device__ __forceinline__ float loss_accumulate(float e, float p, float t)
		{
			if (MODE == kCeFwd)
				return ce_accumulate(e, p, t);
			return __fsub_rn(e, nll_term(p, t));
		}

		template <int MODE>
		__device__ __forceinline__ float loss_gradient(float p, float t, float total_scale)
		{
			if (MODE == kCeBwd)
				return ce_grad(p, t, total_scale);
			return nll_grad(p, t, total_scale);
		}

		// ---- H*W == 1: warp per row. VPL > 0: the row is kept in registers as VPL float4 per lane (C % 4 == 0,
		// aligned rows); VPL == 0: scalar accesses, the row is read again by every pass --------------------
		template <int VPL, int MODE>
		__global__ void __launch_bounds__(256) loss_rows_kernel(const loss_params p)
		{
			const int lane = threadIdx.x & 31;
			const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
			const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
			const int c = p.c;
			for (int64_t row = warp; row < p.rows; row += nwarps)
			{
				const float total_scale = p.mask ? __fmul_rn(p.scale, __ldg(p.mask + row)) : p.scale;
				const float * in = p.in + row * c;
				const float * tg = p.targets + row * c;
				float * out = p.out ? p.out + row * c : nullptr;
				if (VPL > 0)
				{
					constexpr int N = VPL > 0 ? VPL : 1;
					const int c4 = c >> 2;
					const float4 * in4 = reinterpret_cast<const float4 *>(in);
					const float4 * tg4 = reinterpret_cast<const float4 *>(tg);
					float4 * out4 = reinterpret_cast<float4 *>(out);
					float4 v[N], t[N];
					#pragma unroll
					for (int j = 0; j < N; ++j)
					{
						const int idx = j * 32 + lane;
						const bool in_row = idx < c4;
						const float pad = MODE == kFusedFwd ? kLossMaxSeed : 0.0F;
						v[j] = in_row ? ld_stream(in4 + idx) : make_float4(pad, pad, pad, pad);
						t[j] = in_row ? ld_stream(tg4 + idx) : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					}
					if (MODE == kFusedFwd)
					{
						// softmax exactly as softmax_rows_warp4_kernel computes it
						float m = kLossMaxSeed;
						#pragma unroll
						for (int j = 0; j < N; ++j)
							m = loss_ref_max(loss_ref_max(loss_ref_max(loss_ref_max(m, v[j].x), v[j].y), v[j].z), v[j].w);
						m = loss_warp_max(m);
						float s = 0.0F;
						#pragma unroll
						for (int j = 0; j < N; ++j)
							if (j * 32 + lane < c4)
							{
								v[j].x = fast_exp(__fsub_rn(v[j].x, m)); v[j].y = fast_exp(__fsub_rn(v[j].y, m));
								v[j].z = fast_exp(__fsub_rn(v[j].z, m)); v[j].w = fast_exp(__fsub_rn(v[j].w, m));
								s = __fadd_rn(s, __fadd_rn(__fadd_rn(v[j].x, v[j].y), __fadd_rn(v[j].z, v[j].w)));
							}
						s = loss_warp_sum(s);
						const float mult = __fdiv_rn(1.0F, s);
						#pragma unroll
						for (int j = 0; j < N; ++j)
							if (j * 32 + lane < c4)
							{
								v[j] = make_float4(__fmul_rn(v[j].x, mult), __fmul_rn(v[j].y, mult), __fmul_rn(v[j].z, mult), __fmul_rn(v[j].w, mult));
								st_stream(out4 + (j * 32 + lane), v[j]);
							}
					}
					if (MODE == kFusedFwd || MODE == kLossFwd || MODE == kCeFwd)
					{
						float e = 0.0F;
						if (total_scale != 0.0F)
						{
							#pragma unroll
							for (int j = 0; j < N; ++j)
								if (j * 32 + lane < c4)
								{
									e = loss_accumulate<MODE>(e, v[j].x, t[j].x); e = loss_accumulate<MODE>(e, v[j].y, t[j].y);
									e = loss_accumulate<MODE>(e, v[j].z, t[j].z); e = loss_accumulate<MODE>(e, v[j].w, t[j].w);
								}
						}
						e = loss_warp_sum(e);
						if (lane == 0)
							p.err[row] = total_scale != 0.0F ? __fmul_rn(e, total_scale) : 0.0F;
					}
					else
					{
						// gradient of the loss; fused: through the softmax as softmax_rows_warp4_kernel does
						float4 g[N];
						float s = 0.0F;
						#pragma unroll
						for (int j = 0; j < N; ++j)
						{
							g[j] = make_float4(loss_gradient<MODE>(v[j].x, t[j].x, total_scale), loss_gradient<MODE>(v[j].y, t[j].y, total_scale),
								loss_gradient<MODE>(v[j].z, t[j].z, total_scale), loss_gradient<MODE>(v[j].w, t[j].w, total_scale));
							if (MODE == kFusedBwd)
								s = __fadd_rn(s, __fadd_rn(__fadd_rn(__fmul_rn(g[j].x, v[j].x), __fmul_rn(g[j].y, v[j].y)),
									__fadd_rn(__fmul_rn(g[j].z, v[j].z), __fmul_rn(g[j].w, v[j].w))));
						}
						if (MODE == kFusedBwd)
							s = loss_warp_sum(s);
						#pragma unroll
						for (int j = 0; j < N; ++j)
						{
							const int idx = j * 32 + lane;
							if (idx < c4)
							{
								float4 r = g[j];
								if (MODE == kFusedBwd)
									r = make_float4(__fmul_rn(v[j].x, __fsub_rn(g[j].x, s)), __fmul_rn(v[j].y, __fsub_rn(g[j].y, s)),
										__fmul_rn(v[j].z, __fsub_rn(g[j].z, s)), __fmul_rn(v[j].w, __fsub_rn(g[j].w, s)));
								if (p.add)
								{
									const float4 old = out4[idx];
									r = make_float4(__fadd_rn(old.x, r.x), __fadd_rn(old.y, r.y), __fadd_rn(old.z, r.z), __fadd_rn(old.w, r.w));
								}
								st_stream(out4 + idx, r);
							}
						}
					}
				}
				else
				{
					// any C: lanes stride over the row, every pass reads it again
					float mult = 1.0F, m = kLossMaxSeed;
					if (MODE == kFusedFwd)
					{
						for (int f = lane; f < c; f += 32)
							m = loss_ref_max(m, in[f]);
						m = loss_warp_max(m);
						float s = 0.0F;
						for (int f = lane; f < c; f += 32)
							s = __fadd_rn(s, fast_exp(__fsub_rn(in[f], m)));
						s = loss_warp_sum(s);
						mult = __fdiv_rn(1.0F, s);
					}
					if (MODE == kFusedFwd || MODE == kLossFwd || MODE == kCeFwd)
					{
						float e = 0.0F;
						for (int f = lane; f < c; f += 32)
						{
							float pr = in[f];
							if (MODE == kFusedFwd)
							{
								pr = __fmul_rn(fast_exp(__fsub_rn(pr, m)), mult);
								out[f] = pr;
							}
							if (total_scale != 0.0F)
								e = loss_accumulate<MODE>(e, pr, tg[f]);
						}
						e = loss_warp_sum(e);
						if (lane == 0)
							p.err[row] = total_scale != 0.0F ? __fmul_rn(e, total_scale) : 0.0F;
					}
					else
					{
						float s = 0.0F;
						if (MODE == kFusedBwd)
						{
							for (int f = lane; f < c; f += 32)
								s = __fadd_rn(s, __fmul_rn(loss_gradient<MODE>(in[f], tg[f], total_scale), in[f]));
							s = loss_warp_sum(s);
						}
						for (int f = lane; f < c; f += 32)
						{
							const float g = loss_gradient<MODE>(in[f], tg[f], total_scale);
							const float r = MODE == kFusedBwd ? __fmul_rn(in[f], __fsub_rn(g, s)) : g;
							out[f] = p.add ? __fadd_rn(out[f], r) : r;
						}
					}
				}
			}
		}

		// ---- H*W > 1: thread per pixel. CMAX > 0: the column is kept in registers (C <= CMAX); CMAX == 0: any C,
		// every pass reads the column again. Channel order ascending, as in the plain backend ---------------
		// EXACT: the column has exactly CMAX elements; the guards of the unrolled loops fold away at compile time
		template <int CMAX, int MODE, bool EXACT = false>
		__global__ void __launch_bounds__(256) loss_pixels_kernel(const loss_params p)
		{
			const int64_t stride = int64_t(gridDim.x) * blockDim.x;
			const int c = EXACT ? CMAX : p.c;
			const uint32_t hw = p.hw;
			for (int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; q < p.rows; q += stride)
			{
				const uint32_t entry = p.hwdiv.div((uint32_t)q);
				const uint32_t pix = (uint32_t)q - entry * hw;
				const int64_t base = int64_t(entry) * c * hw + pix;
				const float total_scale = p.mask ? __fmul_rn(p.scale, __ldg(p.mask + q)) : p.scale;
				const float * in = p.in + base;
				const float * tg = p.targets + base;
				float * out = p.out ? p.out + base : nullptr;
				constexpr int N = CMAX > 0 ? CMAX : 1;
				float v[N], t[N];
				if (CMAX == 0)
					v[0] = t[0] = 0.0F; // not used without the register copy
				auto value = [&](int f) -> float { return CMAX > 0 ? v[f] : ld_stream(in + int64_t(f) * hw); };
				auto target = [&](int f) -> float { return CMAX > 0 ? t[f] : ld_stream(tg + int64_t(f) * hw); };
				if (CMAX > 0)
				{
					#pragma unroll
					for (int f = 0; f < N; ++f)
					{
						v[f] = f < c ? ld_stream(in + int64_t(f) * hw) : (MODE == kFusedFwd ? kLossMaxSeed : 0.0F);
						t[f] = f < c ? ld_stream(tg + int64_t(f) * hw) : 0.0F;
					}
				}
				if (MODE == kFusedFwd || MODE == kLossFwd || MODE == kCeFwd)
				{
					float m = kLossMaxSeed, mult = 1.0F;
					if (MODE == kFusedFwd)
					{
						// softmax exactly as softmax_pixels_reg_kernel computes it
						float s = 0.0F;
						if (CMAX > 0)
						{
							#pragma unroll
							for (int f = 0; f < N; ++f)
								m = loss_ref_max(m, v[f]);
							#pragma unroll
							for (int f = 0; f < N; ++f)
								if (f < c)
								{
									v[f] = fast_exp(__fsub_rn(v[f], m));
									s = __fadd_rn(s, v[f]);
								}
						}
						else
						{
							for (int f = 0; f < c; ++f)
								m = loss_ref_max(m, value(f));
							for (int f = 0; f < c; ++f)
								s = __fadd_rn(s, fast_exp(__fsub_rn(value(f), m)));
						}
						mult = __fdiv_rn(1.0F, s);
					}
					float e = 0.0F;
					if (CMAX > 0)
					{
						#pragma unroll
						for (int f = 0; f < N; ++f)
							if (f < c)
							{
								float pr = v[f];
								if (MODE == kFusedFwd)
								{
									pr = __fmul_rn(pr, mult);
									out[int64_t(f) * hw] = pr;
								}
								if (total_scale != 0.0F)
									e = loss_accumulate<MODE>(e, pr, t[f]);
							}
					}
					else
					{
						for (int f = 0; f < c; ++f)
						{
							float pr = value(f);
							if (MODE == kFusedFwd)
							{
								pr = __fmul_rn(fast_exp(__fsub_rn(pr, m)), mult);
								out[int64_t(f) * hw] = pr;
							}
							if (total_scale != 0.0F)
								e = loss_accumulate<MODE>(e, pr, target(f));
						}
					}
					p.err[q] = total_scale != 0.0F ? __fmul_rn(e, total_scale) : 0.0F;
				}
				else
				{
					float s = 0.0F;
					if (CMAX > 0)
					{
						// the gradient of the loss takes the place of the target in its register
						#pragma unroll
						for (int f = 0; f < N; ++f)
							if (f < c)
							{
								t[f] = loss_gradient<MODE>(v[f], t[f], total_scale);
								if (MODE == kFusedBwd)
									s = __fadd_rn(s, __fmul_rn(t[f], v[f]));
							}
					}
					else if (MODE == kFusedBwd)
						for (int f = 0; f < c; ++f)
							s = __fadd_rn(s, __fmul_rn(loss_gradient<MODE>(value(f), target(f), total_scale), value(f)));
					auto emit = [&](int f, float pr, float g)
					{
						const float r = MODE == kFusedBwd ? __fmul_rn(pr, __fsub_rn(g, s)) : g;
						float * o = out + int64_t(f) * hw;
						*o = p.add ? __fadd_rn(*o, r) : r;
					};
					if (CMAX > 0)
					{
						#pragma unroll
						for (int f = 0; f < N; ++f)
							if (f < c)
								emit(f, v[f], t[f]);
					}
					else
						for (int f = 0; f < c; ++f)
							emit(f, value(f), loss_gradient<MODE>(value(f), target(f), total_scale));
				}
			}
		}

		template <int MODE>
		int run_loss(cudaStream_t s, const char * who, float * out, float * err, const float * in, const float * targets, const float * mask, float scale,
			int64_t n, int64_t c, int64_t hw, int add)
		{
			if (n < 0 || c <= 0 || hw <= 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: bad extents n=%lld c=%lld hw=%lld", who, (long long)n, (long long)c, (long long)hw);
			if (n == 0)
				return NNF_OK;
			const bool forward = MODE == kFusedFwd || MODE == kLossFwd || MODE == kCeFwd;
			if (!in || !targets || (forward && !err) || (MODE != kLossFwd && MODE != kCeFwd && !out))
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
			if (c > 0x7fffffff || hw > 0x7fffffff)
				return set_error(NNF_ERR_UNSUPPORTED, "%s: extent too large", who);
			loss_params p = {};
			p.scale = scale;
			p.c = (int)c;
			p.add = add;
			if (hw == 1)
			{
				p.out = out; p.err = err; p.in = in; p.targets = targets; p.mask = mask;
				p.rows = n;
				p.hw = 1;
				const int64_t blocks_needed = div_up(n, 8); // 8 warps per CTA
				const int grid = (int)(blocks_needed < int64_t(sm_count()) * 64 ? blocks_needed : int64_t(sm_count()) * 64);
				const bool vec = (c & 3) == 0 && c <= 1024 && aligned16(in) && aligned16(targets) && (!out || aligned16(out));
				if (vec && c <= 128) loss_rows_kernel<1, MODE><<<grid, 256, 0, s>>>(p);
				else if (vec && c <= 256) loss_rows_kernel<2, MODE><<<grid, 256, 0, s>>>(p);
				else if (vec && c <= 512) loss_rows_kernel<4, MODE><<<grid, 256, 0, s>>>(p);
				else if (vec) loss_rows_kernel<8, MODE><<<grid, 256, 0, s>>>(p);
				else loss_rows_kernel<0, MODE><<<grid, 256, 0, s>>>(p);
				return check_launch("loss_rows_kernel");
			}
			const int64_t entries_per_launch = kMaxElemsPerLaunch / hw;
			if (entries_per_launch < 1)
				return set_error(NNF_ERR_UNSUPPORTED, "%s: hw too large", who);
			for (int64_t e0 = 0; e0 < n; e0 += entries_per_launch)
			{
				const int64_t ne = (n - e0 < entries_per_launch) ? (n - e0) : entries_per_launch;
				const int64_t off = e0 * c * hw;
				p.out = out ? out + off : nullptr;
				p.err = err ? err + e0 * hw : nullptr;
				p.in = in + off;
				p.targets = targets + off;
				p.mask = mask ? mask + e0 * hw : nullptr;
				p.rows = ne * hw;
				p.hw = (uint32_t)hw;
				p.hwdiv = fastdiv((uint32_t)hw);
				const int64_t blocks_needed = div_up(p.rows, 256);
				const int grid = (int)(blocks_needed < int64_t(sm_count()) * 128 ? blocks_needed : int64_t(sm_count()) * 128);
				bool launched = false;
				{
					// one instantiation per column length, as in the per-pixel softmax kernel: no dead slots in the unrolled loops
					// and no more registers than the column needs (softmax + loss fused at logits[512,21,128,128]: forward 446 us
					// with 24 slots for 21 elements, 329 us with 21; backward 401 -> 320 us)
#define NNF_EXACT(C) case C: loss_pixels_kernel<C, MODE, true><<<grid, 256, 0, s>>>(p); launched = true; break;
					switch ((int)c)
					{
					NNF_EXACT(2) NNF_EXACT(3) NNF_EXACT(4) NNF_EXACT(5) NNF_EXACT(6) NNF_EXACT(7) NNF_EXACT(8)
					NNF_EXACT(9) NNF_EXACT(10) NNF_EXACT(11) NNF_EXACT(12) NNF_EXACT(13) NNF_EXACT(14) NNF_EXACT(15) NNF_EXACT(16)
					NNF_EXACT(17) NNF_EXACT(18) NNF_EXACT(19) NNF_EXACT(20) NNF_EXACT(21) NNF_EXACT(22) NNF_EXACT(23) NNF_EXACT(24)
					NNF_EXACT(25) NNF_EXACT(26) NNF_EXACT(27) NNF_EXACT(28) NNF_EXACT(29) NNF_EXACT(30) NNF_EXACT(31) NNF_EXACT(32)
					default: break;
					}
#undef NNF_EXACT
				}
				if (launched) {}
				else if (c <= 8) loss_pixels_kernel<8, MODE><<<grid, 256, 0, s>>>(p);
				else if (c <= 16) loss_pixels_kernel<16, MODE><<<grid, 256, 0, s>>>(p);
				else if (c <= 24) loss_pixels_kernel<24, MODE><<<grid, 256, 0, s>>>(p);
				else if (c <= 32) loss_pixels_kernel<32, MODE><<<grid, 256, 0, s>>>(p);
				else loss_pixels_kernel<0, MODE><<<grid, 256, 0, s>>>(p);
				const int st = check_launch("loss_pixels_kernel");
				if (st != NNF_OK)
					return st;
			}
			return NNF_OK;
		}
	}
}

namespace nnf
{
	namespace
	{
		// ---- top-n accuracy (nnforge/plain/accuracy_layer_tester_plain.cpp:64-110, nnforge/cuda/accuracy_layer_tester_cuda.cu) ----
		// The actual class is the first channel with the largest target; rank = channels whose prediction beats that
		// class's (larger, or equal with a smaller index); out[k] = rank <= k ? mask : 0 for k < top_n, out[top_n] = mask.
		struct accuracy_params
		{
			float * out;            // [n][top_n + 1][hw]
			const float * predicted;
			const float * targets;
			const float * mask;     // [n][hw] or null
			int c, top_n;
			int64_t rows;           // H*W == 1: entries; else pixels of this launch
			uint32_t hw;
			fastdiv hwdiv;
		};

		__device__ __forceinline__ void accuracy_emit(const accuracy_params& p, float * out, int64_t plane_stride, int rank, float m)
		{
			for (int k = 0; k < p.top_n; ++k)
				out[k * plane_stride] = rank <= k ? m : 0.0F;
			out[p.top_n * plane_stride] = m;
		}

		// H*W == 1: warp per row
		__global__ void __launch_bounds__(256) accuracy_rows_kernel(const accuracy_params p)
		{
			const int lane = threadIdx.x & 31;
			const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
			const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
			for (int64_t row = warp; row < p.rows; row += nwarps)
			{
				const float m = p.mask ? __ldg(p.mask + row) : 1.0F;
				int rank = 0;
				if (m != 0.0F)
				{
					const float * tg = p.targets + row * p.c;
					const float * pr = p.predicted + row * p.c;
					float best = kLossMaxSeed;
					int cls = -1;
					for (int f = lane; f < p.c; f += 32)
					{
						const float a = ld_stream(tg + f);
						if (a > best)
						{
							best = a;
							cls = f;
						}
					}
					// first channel holding the largest target over the whole row
					#pragma unroll
					for (int o = 16; o > 0; o >>= 1)
					{
						const float ob = __shfl_xor_sync(0xffffffffu, best, o);
						const int oc = __shfl_xor_sync(0xffffffffu, cls, o);
						if (oc >= 0 && (cls < 0 || ob > best || (ob == best && oc < cls)))
						{
							best = ob;
							cls = oc;
						}
					}
					if (cls >= 0)
					{
						const float ref = __ldg(pr + cls);
						int count = 0;
						for (int f = lane; f < p.c; f += 32)
						{
							const float v = ld_stream(pr + f);
							count += (v > ref || (v == ref && f < cls)) ? 1 : 0;
						}
						#pragma unroll
						for (int o = 16; o > 0; o >>= 1)
							count += __shfl_xor_sync(0xffffffffu, count, o);
						rank = count;
					}
				}
				if (lane == 0)
					accuracy_emit(p, p.out + row * (p.top_n + 1), 1, rank, m);
			}
		}

		// H*W > 1: thread per pixel, channels strided by H*W
		__global__ void __launch_bounds__(256) accuracy_pixels_kernel(const accuracy_params p)
		{
			const int64_t stride = int64_t(gridDim.x) * blockDim.x;
			for (int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; q < p.rows; q += stride)
			{
				const uint32_t entry = p.hwdiv.div((uint32_t)q);
				const uint32_t pix = (uint32_t)q - entry * p.hw;
				const int64_t base = int64_t(entry) * p.c * p.hw + pix;
				const float m = p.mask ? __ldg(p.mask + q) : 1.0F;
				int rank = 0;
				if (m != 0.0F)
				{
					float best = kLossMaxSeed;
					int cls = -1;
					for (int f = 0; f < p.c; ++f)
					{
						const float a = ld_stream(p.targets + base + int64_t(f) * p.hw);
						if (a > best)
						{
							best = a;
							cls = f;
						}
					}
					if (cls >= 0)
					{
						const float ref = p.predicted[base + int64_t(cls) * p.hw];
						for (int f = 0; f < p.c; ++f)
						{
							const float v = ld_stream(p.predicted + base + int64_t(f) * p.hw);
							rank += (v > ref || (v == ref && f < cls)) ? 1 : 0;
						}
					}
				}
				accuracy_emit(p, p.out + int64_t(entry) * (p.top_n + 1) * p.hw + pix, p.hw, rank, m);
			}
		}
	}
}

using namespace nnf;

extern "C" int nnf_accuracy_fwd(nnf_stream_t stream, float * out, const float * predicted, const float * targets, const float * mask,
	int top_n, int64_t n, int64_t c, int64_t hw)
{
	if (n < 0 || c <= 0 || hw <= 0 || top_n < 1)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_accuracy_fwd: bad extents n=%lld c=%lld hw=%lld top_n=%d", (long long)n, (long long)c, (long long)hw, top_n);
	if (n == 0)
		return NNF_OK;
	if (!out || !predicted || !targets)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_accuracy_fwd: null pointer");
	if (c > 0x7fffffff || hw > 0x7fffffff)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_accuracy_fwd: extent too large");
	cudaStream_t s = (cudaStream_t)stream;
	accuracy_params p = {};
	p.c = (int)c;
	p.top_n = top_n;
	if (hw == 1)
	{
		p.out = out; p.predicted = predicted; p.targets = targets; p.mask = mask;
		p.rows = n;
		p.hw = 1;
		const int64_t blocks_needed = div_up(n, 8);
		const int grid = (int)(blocks_needed < int64_t(sm_count()) * 64 ? blocks_needed : int64_t(sm_count()) * 64);
		accuracy_rows_kernel<<<grid, 256, 0, s>>>(p);
		return check_launch("accuracy_rows_kernel");
	}
	const int64_t entries_per_launch = kMaxElemsPerLaunch / hw;
	if (entries_per_launch < 1)
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_accuracy_fwd: hw too large");
	for (int64_t e0 = 0; e0 < n; e0 += entries_per_launch)
	{
		const int64_t ne = (n - e0 < entries_per_launch) ? (n - e0) : entries_per_launch;
		p.out = out + e0 * (top_n + 1) * hw;
		p.predicted = predicted + e0 * c * hw;
		p.targets = targets + e0 * c * hw;
		p.mask = mask ? mask + e0 * hw : nullptr;
		p.rows = ne * hw;
		p.hw = (uint32_t)hw;
		p.hwdiv = fastdiv((uint32_t)hw);
		const int64_t blocks_needed = div_up(p.rows, 256);
		const int grid = (int)(blocks_needed < int64_t(sm_count()) * 128 ? blocks_needed : int64_t(sm_count()) * 128);
		accuracy_pixels_kernel<<<grid, 256, 0, s>>>(p);
		const int st = check_launch("accuracy_pixels_kernel");
		if (st != NNF_OK)
			return st;
	}
	return NNF_OK;
}

extern "C" int nnf_softmax_nll_fwd(nnf_stream_t stream, float * probs, float * err, const float * logits, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw)
{
	return run_loss<kFusedFwd>((cudaStream_t)stream, "nnf_softmax_nll_fwd", probs, err, logits, targets, mask, scale, n, c, hw, 0);
}

extern "C" int nnf_softmax_nll_bwd(nnf_stream_t stream, float * dlogits, const float * probs, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	return run_loss<kFusedBwd>((cudaStream_t)stream, "nnf_softmax_nll_bwd", dlogits, nullptr, probs, targets, mask, scale, n, c, hw, add_to_destination ? 1 : 0);
}

extern "C" int nnf_nll_fwd(nnf_stream_t stream, float * err, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw)
{
	return run_loss<kLossFwd>((cudaStream_t)stream, "nnf_nll_fwd", nullptr, err, predicted, targets, mask, scale, n, c, hw, 0);
}

extern "C" int nnf_cross_entropy_fwd(nnf_stream_t stream, float * err, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw)
{
	return run_loss<kCeFwd>((cudaStream_t)stream, "nnf_cross_entropy_fwd", nullptr, err, predicted, targets, mask, scale, n, c, hw, 0);
}

extern "C" int nnf_cross_entropy_bwd(nnf_stream_t stream, float * dpredicted, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	return run_loss<kCeBwd>((cudaStream_t)stream, "nnf_cross_entropy_bwd", dpredicted, nullptr, predicted, targets, mask, scale, n, c, hw, add_to_destination ? 1 : 0);
}

extern "C" int nnf_nll_bwd(nnf_stream_t stream, float * dpredicted, const float * predicted, const float * targets, const float * mask,
	float scale, int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	return run_loss<kLossBwd>((cudaStream_t)stream, "nnf_nll_bwd", dpredicted, nullptr, predicted, targets, mask, scale, n, c, hw, add_to_destination ? 1 : 0);
}
