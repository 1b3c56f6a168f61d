// average_subsampling over the two spatial dimensions (non-overlapping windows, stride = window), stand-alone and
// fused behind batch norm -> residual add -> ReLU: the global average pooling in front of a classifier is the
// case win = (W, H). Semantics of nnforge/plain/average_subsampling_layer_tester_plain.cpp:120-135 and
// average_subsampling_layer_updater_plain.cpp:270-285:
//   forward : out = (sum over the window, x fastest then y, starting from +0) * mult
//   backward: dx  = dy[window of the element] * mult
// mult is the layer's effective alpha (1 / window elements unless the layer sets alpha). The sum of a window is
// taken sequentially in the plain backend's order by one thread, so the result is bit-exact.
//
// Forward: a CTA stages a group of whole planes in shared memory with coalesced 128-bit accesses (applying the fused
// per-element chain and writing z when fused), then one thread per output walks its window in shared memory.
// Backward is a streaming pass: every element fetches its window's gradient (a small, cached tensor).
#include "nnf_common.cuh"

namespace nnf
{
	namespace
	{
		constexpr int kAvgThreads = 256;
		constexpr int kAvgMaxGroup = 512;

		struct avg_params
		{
			const float * x;        // input (forward) / unused (backward)
			const float * res;      // fused forward: residual or null
			float * z;              // fused forward: relu(bn(x) + res), written
			const float * zin;      // fused backward: the same tensor, read
			float * pooled;         // forward output [planes][oh][ow]
			const float * dpooled;  // backward input
			float * dx;             // backward output (fused: gradient towards the batch-norm input)
			float * dres;           // fused backward: gradient towards the residual input, or null
			const float * gamma, * beta, * mean, * invsigma; // fused; gamma null: no batch norm
			float slope, mult;
			int add;                // stand-alone backward: accumulate into dx
			int64_t planes;
			uint32_t c, h, w, hw, win_w, win_h, oh, ow, ohw;
			uint32_t group;         // planes per CTA iteration
			int vec_ok;
			fastdiv d_hw, d_w, d_c, d_ohw, d_ow, d_win_w, d_win_h;
		};

		template <bool FUSED>
		__global__ void __launch_bounds__(kAvgThreads) avgpool_fwd_kernel(const avg_params p)
		{
			extern __shared__ float s_z[];
			__shared__ float s_mult[FUSED ? kAvgMaxGroup : 1];
			__shared__ float s_add[FUSED ? kAvgMaxGroup : 1];
			const bool has_bn = FUSED && p.gamma != nullptr;
			const bool has_res = FUSED && p.res != nullptr;
			const int64_t ngroups = (p.planes + p.group - 1) / p.group;
			for (int64_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x)
			{
				const int64_t plane0 = grp * p.group;
				const uint32_t np = (uint32_t)((p.planes - plane0 < p.group) ? (p.planes - plane0) : p.group);
				const uint32_t count = np * p.hw;
				const int64_t base = plane0 * p.hw;
				if (has_bn)
				{
					// batch-norm scale/shift of each plane of the group (batch_norm_layer_tester_plain.cpp:60-61)
					const uint32_t ch0 = (uint32_t)(plane0 - int64_t(p.d_c.div((uint32_t)plane0)) * p.c);
					for (uint32_t lp = threadIdx.x; lp < np; lp += kAvgThreads)
					{
						uint32_t channel = ch0 + lp;
						channel -= p.d_c.div(channel) * p.c;
						const float mult = __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel));
						s_mult[lp] = mult;
						s_add[lp] = __fsub_rn(__ldg(p.beta + channel), __fmul_rn(mult, __ldg(p.mean + channel)));
					}
				}
				__syncthreads(); // also: the previous group's windows have been read
				auto fused = [&](float mult, float add, float v, float r) -> float
				{
					if (!FUSED)
						return v;
					float t = v;
					if (has_bn)
						t = __fadd_rn(__fmul_rn(v, mult), add);
					if (has_res)
						t = __fadd_rn(__fadd_rn(0.0F, t), r); // add layer, alpha = 1: (0 + bn) + residual
					return t >= 0.0F ? t : __fmul_rn(t, p.slope);
				};
				const uint32_t nvec = (p.vec_ok && (base & 3) == 0) ? (count >> 2) : 0;
				// independent 128-bit loads per thread before any is consumed: the stand-alone layer reads one tensor and needs
				// them to cover the latency (7x7 global pooling 35 -> 27 us); the fused form has two input streams and a store
				// per vector already and is slower with more (14x14: 119 -> 143 us)
				constexpr int kInFlight = FUSED ? 1 : 4;
				for (uint32_t v0 = threadIdx.x; v0 < nvec; v0 += kAvgThreads * kInFlight)
				{
				float4 av[kInFlight], rv[kInFlight];
				#pragma unroll
				for (int u = 0; u < kInFlight; ++u)
				{
					const uint32_t v = v0 + u * kAvgThreads;
					rv[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					if (v < nvec)
					{
						av[u] = ld_stream(reinterpret_cast<const float4 *>(p.x + base) + v);
						if (has_res)
							rv[u] = ld_stream(reinterpret_cast<const float4 *>(p.res + base) + v);
					}
				}
				#pragma unroll
				for (int u = 0; u < kInFlight; ++u)
				{
					const uint32_t v = v0 + u * kAvgThreads;
					if (v >= nvec)
						break;
					const float4 a = av[u];
					const float4 r = rv[u];
					// a vector lies in one plane unless it straddles a plane boundary (H*W not a multiple of 4)
					float m0 = 1.0F, a0 = 0.0F, m1 = 1.0F, a1 = 0.0F;
					uint32_t left = 4;
					if (has_bn)
					{
						const uint32_t lp0 = p.d_hw.div(v << 2);
						left = (lp0 + 1) * p.hw - (v << 2);
						const uint32_t lp1 = left >= 4 ? lp0 : lp0 + 1;
						m0 = s_mult[lp0]; a0 = s_add[lp0];
						m1 = s_mult[lp1]; a1 = s_add[lp1];
					}
					const float4 o = make_float4(fused(m0, a0, a.x, r.x), fused(left > 1 ? m0 : m1, left > 1 ? a0 : a1, a.y, r.y),
						fused(left > 2 ? m0 : m1, left > 2 ? a0 : a1, a.z, r.z), fused(left > 3 ? m0 : m1, left > 3 ? a0 : a1, a.w, r.w));
					if (FUSED)
						st_stream(reinterpret_cast<float4 *>(p.z + base) + v, o);
					reinterpret_cast<float4 *>(s_z)[v] = o;
				}
				}
				for (uint32_t e = (nvec << 2) + threadIdx.x; e < count; e += kAvgThreads)
				{
					const uint32_t lp = has_bn ? p.d_hw.div(e) : 0;
					const float o = fused(has_bn ? s_mult[lp] : 1.0F, has_bn ? s_add[lp] : 0.0F, p.x[base + e], has_res ? p.res[base + e] : 0.0F);
					if (FUSED)
						p.z[base + e] = o;
					s_z[e] = o;
				}
				__syncthreads();
				const uint32_t nout = np * p.ohw;
				for (uint32_t o = threadIdx.x; o < nout; o += kAvgThreads)
				{
					const uint32_t lp = p.d_ohw.div(o);
					const uint32_t rem = o - lp * p.ohw;
					const uint32_t oy = p.d_ow.div(rem);
					const uint32_t ox = rem - oy * p.ow;
					const float * win = s_z + lp * p.hw + oy * p.win_h * p.w + ox * p.win_w;
					// the window in the plain backend's order (rows, then columns). The stand-alone layer fetches eight values
					// before it adds them one by one, so that the chain of additions does not wait for shared memory at every
					// step (14x14 global pooling 85 -> 74 us); the fused kernel is slower with it (more registers: 119 -> 127 us)
					constexpr int kFetch = FUSED ? 1 : 8;
					float sum = 0.0F;
					for (uint32_t y = 0; y < p.win_h; ++y)
					{
						const float * row = win + y * p.w;
						for (uint32_t x0 = 0; x0 < p.win_w; x0 += kFetch)
						{
							float t[kFetch];
							#pragma unroll
							for (int u = 0; u < kFetch; ++u)
								t[u] = (x0 + u < p.win_w) ? row[x0 + u] : 0.0F;
							#pragma unroll
							for (int u = 0; u < kFetch; ++u)
								if (x0 + u < p.win_w)
									sum = __fadd_rn(sum, t[u]);
						}
					}
					p.pooled[plane0 * p.ohw + o] = __fmul_rn(sum, p.mult);
				}
			}
		}

		// 2x2 windows on rows of whole float4s (stand-alone layer): a thread reads the same float4 column of the two input
		// rows of an output row and writes two outputs; each window is summed in the plain backend's order
		// (((0 + x00) + x01) + x10) + x11. No shared memory, every access 8 or 16 bytes wide.
		__global__ void __launch_bounds__(kAvgThreads) avgpool_fwd_2x2_kernel(float * pooled, const float * x, int64_t out_rows, uint32_t w4, fastdiv d_w4, float mult)
		{
			const int64_t total = out_rows * w4;
			const int64_t stride = int64_t(gridDim.x) * kAvgThreads * 2;
			for (int64_t i0 = int64_t(blockIdx.x) * kAvgThreads * 2 + threadIdx.x; i0 < total; i0 += stride)
			{
				float4 a[2], b[2];
				int64_t row[2];
				uint32_t col[2];
				#pragma unroll
				for (int u = 0; u < 2; ++u)
				{
					const int64_t i = i0 + int64_t(u) * kAvgThreads;
					if (i < total)
					{
						// out_rows * w4 < 2^31 per launch (checked by the caller)
						row[u] = d_w4.div((uint32_t)i);
						col[u] = (uint32_t)(i - row[u] * w4);
						const float4 * in = reinterpret_cast<const float4 *>(x) + row[u] * 2 * w4 + col[u];
						a[u] = ld_stream(in);
						b[u] = ld_stream(in + w4);
					}
				}
				#pragma unroll
				for (int u = 0; u < 2; ++u)
				{
					const int64_t i = i0 + int64_t(u) * kAvgThreads;
					if (i < total)
					{
						const float s0 = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(0.0F, a[u].x), a[u].y), b[u].x), b[u].y);
						const float s1 = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(0.0F, a[u].z), a[u].w), b[u].z), b[u].w);
						__stcs(reinterpret_cast<float2 *>(pooled) + row[u] * w4 + col[u], make_float2(__fmul_rn(s0, mult), __fmul_rn(s1, mult)));
					}
				}
			}
		}

		// the same for rows of whole float2s only (14x14): one output per thread
		__global__ void __launch_bounds__(kAvgThreads) avgpool_fwd_2x2_pair_kernel(float * pooled, const float * x, int64_t out_rows, uint32_t w2, fastdiv d_w2, float mult)
		{
			const int64_t total = out_rows * w2;
			const int64_t stride = int64_t(gridDim.x) * kAvgThreads * 4;
			for (int64_t i0 = int64_t(blockIdx.x) * kAvgThreads * 4 + threadIdx.x; i0 < total; i0 += stride)
			{
				float2 a[4], b[4];
				#pragma unroll
				for (int u = 0; u < 4; ++u)
				{
					const int64_t i = i0 + int64_t(u) * kAvgThreads;
					if (i < total)
					{
						const int64_t row = d_w2.div((uint32_t)i);
						const float2 * in = reinterpret_cast<const float2 *>(x) + row * 2 * w2 + (i - row * w2);
						a[u] = __ldcs(in);
						b[u] = __ldcs(in + w2);
					}
				}
				#pragma unroll
				for (int u = 0; u < 4; ++u)
				{
					const int64_t i = i0 + int64_t(u) * kAvgThreads;
					if (i < total)
						__stcs(pooled + i, __fmul_rn(__fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(0.0F, a[u].x), a[u].y), b[u].x), b[u].y), mult));
				}
			}
		}

		// backward of the 2x2 stand-alone layer on rows of whole float2s: every element of a window receives dy * mult
		// (average_subsampling_layer_updater_plain.cpp:270-285); a thread takes one gradient and writes, or accumulates
		// into, the two float2s of its window
		__global__ void __launch_bounds__(kAvgThreads) avgpool_bwd_2x2_pair_kernel(float * dx, const float * dy, int64_t out_rows, uint32_t w2, fastdiv d_w2, float mult, int add)
		{
			const int64_t total = out_rows * w2;
			const int64_t stride = int64_t(gridDim.x) * kAvgThreads * 4;
			for (int64_t i0 = int64_t(blockIdx.x) * kAvgThreads * 4 + threadIdx.x; i0 < total; i0 += stride)
			{
				float g[4];
				#pragma unroll
				for (int u = 0; u < 4; ++u)
				{
					const int64_t i = i0 + int64_t(u) * kAvgThreads;
					if (i < total)
						g[u] = __ldcs(dy + i);
				}
				#pragma unroll
				for (int u = 0; u < 4; ++u)
				{
					const int64_t i = i0 + int64_t(u) * kAvgThreads;
					if (i < total)
					{
						const int64_t row = d_w2.div((uint32_t)i);
						float2 * out = reinterpret_cast<float2 *>(dx) + row * 2 * w2 + (i - row * w2);
						const float err = __fmul_rn(g[u], mult);
						float2 top = make_float2(err, err), bottom = make_float2(err, err);
						if (add)
						{
							const float2 t = out[0], b = out[w2];
							top = make_float2(__fadd_rn(t.x, err), __fadd_rn(t.y, err));
							bottom = make_float2(__fadd_rn(b.x, err), __fadd_rn(b.y, err));
						}
						__stcs(out, top);
						__stcs(out + w2, bottom);
					}
				}
			}
		}

		// planes too large for shared memory: one thread per output reads its window from global memory
		__global__ void __launch_bounds__(kAvgThreads) avgpool_fwd_direct_kernel(const avg_params p)
		{
			const int64_t total = p.planes * p.ohw;
			const int64_t stride = int64_t(gridDim.x) * kAvgThreads;
			for (int64_t o = int64_t(blockIdx.x) * kAvgThreads + threadIdx.x; o < total; o += stride)
			{
				const int64_t plane = o / p.ohw;
				const uint32_t rem = (uint32_t)(o - plane * p.ohw);
				const uint32_t oy = p.d_ow.div(rem);
				const uint32_t ox = rem - oy * p.ow;
				const float * win = p.x + plane * p.hw + size_t(oy) * p.win_h * p.w + ox * p.win_w;
				float sum = 0.0F;
				for (uint32_t y = 0; y < p.win_h; ++y)
					for (uint32_t x = 0; x < p.win_w; ++x)
						sum = __fadd_rn(sum, win[size_t(y) * p.w + x]);
				p.pooled[o] = __fmul_rn(sum, p.mult);
			}
		}

		template <bool FUSED>
		__global__ void __launch_bounds__(kAvgThreads) avgpool_bwd_kernel(const avg_params p, int64_t base, uint32_t count)
		{
			// elements [base, base + count) of the input-sized tensors; base is a multiple of hw
			const int64_t plane_base = base / p.hw;
			// position of an element inside the launch: plane (relative), row, column; advanced element by element
			struct cursor
			{
				uint32_t lp, iy, ix;
			};
			auto locate = [&](uint32_t e) -> cursor
			{
				cursor k;
				k.lp = p.d_hw.div(e);
				const uint32_t rem = e - k.lp * p.hw;
				k.iy = p.d_w.div(rem);
				k.ix = rem - k.iy * p.w;
				return k;
			};
			auto advance = [&](cursor& k)
			{
				if (++k.ix == p.w)
				{
					k.ix = 0;
					if (++k.iy == p.h)
					{
						k.iy = 0;
						++k.lp;
					}
				}
			};
			auto plane_factor = [&](uint32_t lp) -> float
			{
				if (!FUSED || !p.gamma)
					return 1.0F;
				const int64_t plane = plane_base + lp;
				const uint32_t channel = (uint32_t)(plane - int64_t(p.d_c.div((uint32_t)plane)) * p.c);
				return __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel));
			};
			auto element = [&](const cursor& k, float factor, float zval, float old, float& odx, float& ores)
			{
				const int64_t plane = plane_base + k.lp;
				const float dz = __fmul_rn(__ldg(p.dpooled + plane * p.ohw + p.d_win_h.div(k.iy) * p.ow + p.d_win_w.div(k.ix)), p.mult);
				if (FUSED)
				{
					// ReLU gate from the sign bit of z; add layer backward with alpha 1 is the identity; frozen batch
					// norm scales by gamma*invsigma
					const float ds = (__float_as_uint(zval) >> 31) ? __fmul_rn(dz, p.slope) : dz;
					ores = ds;
					odx = p.gamma ? __fmul_rn(ds, factor) : ds;
				}
				else
					odx = p.add ? __fadd_rn(old, dz) : dz;
			};
			const uint32_t stride = gridDim.x * kAvgThreads;
			const uint32_t nvec = p.vec_ok ? (count >> 2) : 0;
			for (uint32_t v = blockIdx.x * kAvgThreads + threadIdx.x; v < nvec; v += stride)
			{
				float4 z4 = make_float4(0.0F, 0.0F, 0.0F, 0.0F), old = z4, ox, orr;
				if (FUSED)
					z4 = ld_stream(reinterpret_cast<const float4 *>(p.zin + base) + v);
				else if (p.add)
					old = ld_stream(reinterpret_cast<const float4 *>(p.dx + base) + v);
				cursor k = locate(v << 2);
				const uint32_t lp0 = k.lp;
				const float f0 = plane_factor(lp0);
				float f1 = f0;
				if ((lp0 + 1) * p.hw - (v << 2) < 4) // the vector straddles a plane boundary
					f1 = plane_factor(lp0 + 1);
				element(k, f0, z4.x, old.x, ox.x, orr.x);
				advance(k);
				element(k, k.lp == lp0 ? f0 : f1, z4.y, old.y, ox.y, orr.y);
				advance(k);
				element(k, k.lp == lp0 ? f0 : f1, z4.z, old.z, ox.z, orr.z);
				advance(k);
				element(k, k.lp == lp0 ? f0 : f1, z4.w, old.w, ox.w, orr.w);
				if (p.dx)
					st_stream(reinterpret_cast<float4 *>(p.dx + base) + v, ox);
				if (FUSED && p.dres)
					st_stream(reinterpret_cast<float4 *>(p.dres + base) + v, orr);
			}
			for (uint32_t e = (nvec << 2) + blockIdx.x * kAvgThreads + threadIdx.x; e < count; e += stride)
			{
				float odx, ores;
				const cursor k = locate(e);
				element(k, plane_factor(k.lp), FUSED ? p.zin[base + e] : 0.0F, (!FUSED && p.add) ? p.dx[base + e] : 0.0F, odx, ores);
				if (p.dx)
					p.dx[base + e] = odx;
				if (FUSED && p.dres)
					p.dres[base + e] = ores;
			}
		}

		int make_avg(avg_params& p, const char * who, int64_t n, int64_t c, int64_t h, int64_t w, int win_w, int win_h, float mult)
		{
			if (n < 0 || c <= 0 || h <= 0 || w <= 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: bad extents n=%lld c=%lld h=%lld w=%lld", who, (long long)n, (long long)c, (long long)h, (long long)w);
			if (win_w < 1 || win_h < 1 || w % win_w != 0 || h % win_h != 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: the window %dx%d must divide the plane %lldx%lld", who, win_w, win_h, (long long)w, (long long)h);
			if (h * w > 0x7fffffff || c > 0x7fffffff || n * c > 0x7fffffff)
				return set_error(NNF_ERR_UNSUPPORTED, "%s: extent too large", who);
			p.planes = n * c;
			p.c = (uint32_t)c; p.h = (uint32_t)h; p.w = (uint32_t)w; p.hw = (uint32_t)(h * w);
			p.win_w = (uint32_t)win_w; p.win_h = (uint32_t)win_h;
			p.oh = (uint32_t)(h / win_h); p.ow = (uint32_t)(w / win_w); p.ohw = p.oh * p.ow;
			p.mult = mult;
			p.d_hw = fastdiv(p.hw); p.d_w = fastdiv(p.w); p.d_c = fastdiv(p.c); p.d_ohw = fastdiv(p.ohw); p.d_ow = fastdiv(p.ow);
			p.d_win_w = fastdiv(p.win_w); p.d_win_h = fastdiv(p.win_h);
			return NNF_OK;
		}

		int run_avg_fwd(cudaStream_t s, bool fused, avg_params& p)
		{
			if (p.planes == 0)
				return NNF_OK;
			if (!fused && p.win_w == 2 && p.win_h == 2 && p.w % 4 == 0 && p.h % 2 == 0 && aligned16(p.x) && (reinterpret_cast<uintptr_t>(p.pooled) & 7) == 0
				&& p.planes * p.oh * (p.w / 4) < (int64_t(1) << 31))
			{
				const int64_t out_rows = p.planes * p.oh;
				const uint32_t w4 = p.w / 4;
				const int64_t blocks = div_up(out_rows * w4, kAvgThreads * 2);
				const int grid = (int)(blocks < int64_t(sm_count()) * 64 ? blocks : int64_t(sm_count()) * 64);
				avgpool_fwd_2x2_kernel<<<grid, kAvgThreads, 0, s>>>(p.pooled, p.x, out_rows, w4, fastdiv(w4), p.mult);
				return check_launch("avgpool_fwd_2x2_kernel");
			}
			if (!fused && p.win_w == 2 && p.win_h == 2 && p.w % 2 == 0 && p.h % 2 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 7) == 0
				&& p.planes * p.oh * (p.w / 2) < (int64_t(1) << 31))
			{
				const int64_t out_rows = p.planes * p.oh;
				const uint32_t w2 = p.w / 2;
				const int64_t blocks = div_up(out_rows * w2, kAvgThreads * 4);
				const int grid = (int)(blocks < int64_t(sm_count()) * 64 ? blocks : int64_t(sm_count()) * 64);
				avgpool_fwd_2x2_pair_kernel<<<grid, kAvgThreads, 0, s>>>(p.pooled, p.x, out_rows, w2, fastdiv(w2), p.mult);
				return check_launch("avgpool_fwd_2x2_pair_kernel");
			}
			const size_t plane_bytes = size_t(p.hw) * sizeof(float);
			int64_t group = int64_t(16 * 1024 / plane_bytes);
			if (group < 1) group = 1;
			if (group > kAvgMaxGroup) group = kAvgMaxGroup;
			if (group > p.planes) group = p.planes;
			// planes that are not whole float4s (7x7): a group of a multiple of 4 / gcd(H*W, 4) planes still starts and
			// ends on a vector boundary, so the vector path below applies to every group
			const int64_t unit = (p.hw % 4 == 0) ? 1 : ((p.hw % 2 == 0) ? 2 : 4);
			if (group > unit)
				group -= group % unit;
			const size_t smem = size_t(group) * plane_bytes;
			if (smem > staging_smem_limit())
			{
				if (fused)
					return set_error(NNF_ERR_UNSUPPORTED, "fused average pooling needs planes of at most %zu bytes", staging_smem_limit());
				const int64_t blocks = div_up(p.planes * p.ohw, kAvgThreads);
				avgpool_fwd_direct_kernel<<<(int)(blocks < int64_t(sm_count()) * 8 ? blocks : int64_t(sm_count()) * 8), kAvgThreads, 0, s>>>(p);
				return check_launch("avgpool_fwd_direct_kernel");
			}
			p.group = (uint32_t)group;
			p.vec_ok = ((group * p.hw) % 4 == 0 && aligned16(p.x) && (!p.res || aligned16(p.res)) && (!p.z || aligned16(p.z))) ? 1 : 0;
			const int64_t ngroups = div_up(p.planes, group);
			int per_sm = (int)(staging_smem_limit() / (smem + 4096 + 1024));
			per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
			const int64_t cap = int64_t(sm_count()) * per_sm * 4;
			const int grid = (int)(ngroups < cap ? ngroups : cap);
			cudaError_t e;
			if (fused)
			{
				e = cudaFuncSetAttribute(avgpool_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit());
				if (e == cudaSuccess)
					avgpool_fwd_kernel<true><<<grid, kAvgThreads, smem, s>>>(p);
			}
			else
			{
				e = cudaFuncSetAttribute(avgpool_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit());
				if (e == cudaSuccess)
					avgpool_fwd_kernel<false><<<grid, kAvgThreads, smem, s>>>(p);
			}
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
			return check_launch("avgpool_fwd_kernel");
		}

		int run_avg_bwd(cudaStream_t s, bool fused, avg_params& p)
		{
			const int64_t total = p.planes * p.hw;
			if (total == 0)
				return NNF_OK;
			if (!fused && p.win_w == 2 && p.win_h == 2 && p.w % 2 == 0 && p.h % 2 == 0 && p.dx && (reinterpret_cast<uintptr_t>(p.dx) & 7) == 0
				&& p.planes * p.oh * (p.w / 2) < (int64_t(1) << 31))
			{
				const int64_t out_rows = p.planes * p.oh;
				const uint32_t w2 = p.w / 2;
				const int64_t blocks = div_up(out_rows * w2, kAvgThreads * 4);
				const int grid = (int)(blocks < int64_t(sm_count()) * 64 ? blocks : int64_t(sm_count()) * 64);
				avgpool_bwd_2x2_pair_kernel<<<grid, kAvgThreads, 0, s>>>(p.dx, p.dpooled, out_rows, w2, fastdiv(w2), p.mult, p.add);
				return check_launch("avgpool_bwd_2x2_pair_kernel");
			}
			p.vec_ok = ((!p.dx || aligned16(p.dx)) && (!fused || (aligned16(p.zin) && (!p.dres || aligned16(p.dres))))) ? 1 : 0;
			// launches of at most 2^31 elements, split at plane boundaries (and at multiples of 4 elements for the vector path)
			int64_t planes_per_launch = kMaxElemsPerLaunch / p.hw;
			if (planes_per_launch < 1)
				return set_error(NNF_ERR_UNSUPPORTED, "average pooling backward: plane too large");
			if (planes_per_launch > 4)
				planes_per_launch &= ~int64_t(3);
			for (int64_t pl = 0; pl < p.planes; pl += planes_per_launch)
			{
				const int64_t np = (p.planes - pl < planes_per_launch) ? (p.planes - pl) : planes_per_launch;
				const int64_t base = pl * p.hw;
				const uint32_t count = (uint32_t)(np * p.hw);
				avg_params q = p;
				if ((base & 3) != 0)
					q.vec_ok = 0;
				const int64_t blocks = div_up(int64_t(count) / 4 + 1, kAvgThreads);
				const int grid = (int)(blocks < int64_t(sm_count()) * 64 ? blocks : int64_t(sm_count()) * 64);
				if (fused)
					avgpool_bwd_kernel<true><<<grid, kAvgThreads, 0, s>>>(q, base, count);
				else
					avgpool_bwd_kernel<false><<<grid, kAvgThreads, 0, s>>>(q, base, count);
				const int st = check_launch("avgpool_bwd_kernel");
				if (st != NNF_OK)
					return st;
			}
			return NNF_OK;
		}
	}
}

using namespace nnf;

extern "C" int nnf_avgpool_fwd(nnf_stream_t stream, float * y, const float * x, int64_t n, int64_t c, int64_t h, int64_t w,
	int win_w, int win_h, float mult)
{
	avg_params p = {};
	int st = make_avg(p, "nnf_avgpool_fwd", n, c, h, w, win_w, win_h, mult);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!y || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_avgpool_fwd: null pointer");
	p.x = x; p.pooled = y;
	return run_avg_fwd((cudaStream_t)stream, false, p);
}

extern "C" int nnf_avgpool_bwd(nnf_stream_t stream, float * dx, const float * dy, int64_t n, int64_t c, int64_t h, int64_t w,
	int win_w, int win_h, float mult, int add_to_destination)
{
	avg_params p = {};
	int st = make_avg(p, "nnf_avgpool_bwd", n, c, h, w, win_w, win_h, mult);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!dx || !dy)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_avgpool_bwd: null pointer");
	p.dx = dx; p.dpooled = dy; p.add = add_to_destination ? 1 : 0;
	return run_avg_bwd((cudaStream_t)stream, false, p);
}

extern "C" int nnf_bn_add_relu_avgpool_fwd(nnf_stream_t stream, float * z, float * pooled, const float * x, const float * residual,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	float relu_slope, int64_t n, int64_t c, int64_t h, int64_t w, int win_w, int win_h, float mult)
{
	avg_params p = {};
	int st = make_avg(p, "nnf_bn_add_relu_avgpool_fwd", n, c, h, w, win_w, win_h, mult);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!z || !pooled || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_avgpool_fwd: null pointer");
	if (gamma && (!beta || !mean || !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_avgpool_fwd: gamma given but beta/mean/invsigma missing");
	p.x = x; p.res = residual; p.z = z; p.pooled = pooled;
	p.gamma = gamma; p.beta = beta; p.mean = mean; p.invsigma = invsigma;
	p.slope = relu_slope;
	return run_avg_fwd((cudaStream_t)stream, true, p);
}

extern "C" int nnf_bn_add_relu_avgpool_bwd(nnf_stream_t stream, float * dx, float * dresidual, const float * dpooled, const float * z,
	const float * gamma, const float * invsigma, float relu_slope,
	int64_t n, int64_t c, int64_t h, int64_t w, int win_w, int win_h, float mult)
{
	avg_params p = {};
	int st = make_avg(p, "nnf_bn_add_relu_avgpool_bwd", n, c, h, w, win_w, win_h, mult);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if ((!dx && !dresidual) || !dpooled || !z)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_avgpool_bwd: null pointer");
	if (gamma && !invsigma)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_avgpool_bwd: gamma given but invsigma missing");
	p.dx = dx; p.dres = dresidual; p.dpooled = dpooled; p.zin = z;
	p.gamma = gamma; p.invsigma = invsigma;
	p.slope = relu_slope;
	return run_avg_bwd((cudaStream_t)stream, true, p);
}
