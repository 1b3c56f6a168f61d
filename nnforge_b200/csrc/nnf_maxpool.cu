// 2-D max subsampling forward/backward, stand-alone and fused behind batch norm -> residual add ->
// ReLU (the tail of a ResNet block). HBM-bound.
//
// Data movement: a CTA owns a group of whole consecutive (n, c) planes, which are contiguous in the
// planar layout. Forward: the group is read once with coalesced 128-bit loads, the fused
// per-element result z is written straight back (it is needed by later layers and by backward) and
// also kept in shared memory; the overlapping windows are then evaluated from shared memory and the
// pooled values + argmax are written with coalesced stores. Every HBM byte is touched once:
//   forward  bytes per input element = 4*(inputs) + 4 (z, fused only) + 8*rho   (rho = out/in pixels)
// Backward is a gather: the group's pooled gradients and argmax are staged in shared memory and
// every input element sums the few windows that cover it and whose argmax points at it, in ascending
// output index - the order in which nnForge's plain backend scatters them serially
// (nnforge/plain/max_subsampling_layer_updater_plain.cpp:201-229) - so the result is deterministic and
// bit-identical to that order, with no zero-fill pass and no atomics.
//
// Tie-break and argmax format are the plain backend's: window scanned x-fastest, the first element
// seeds, a later one wins only on a strict compare; argmax = absolute input element offset (uint32)
// (nnforge/plain/max_subsampling_layer_updater_plain.cpp:139-159). round_up clips the last window.
// Planes too large for shared memory fall back to direct global-memory kernels.
#include "nnf_common.cuh"

#include <stdlib.h>

namespace nnf
{
	namespace
	{
		constexpr int kThreads = 256;
		constexpr int64_t kGroupFloats = 8192;       // target staged floats per CTA iteration (32 KB)

		struct pool_geom
		{
			uint32_t c, h, w, hw, oh, ow, ohw;
			int win_w, win_h, sw, sh;
			int is_min;
			fastdiv d_w, d_hw, d_ow, d_ohw, d_sw, d_sh, d_c;
		};

		struct pool_fwd_params
		{
			pool_geom g;
			float * z;             // fused only: per-element result written back
			float * pooled;
			uint32_t * argmax;     // may be null
			const float * x;
			const float * res;     // fused only
			const float * gamma;   // null -> no batch norm
			const float * beta;
			const float * mean;
			const float * invsigma;
			float slope;
			int64_t planes;
			int group;             // planes per CTA iteration
			int vec_ok;
		};

		// Scans one window of plane `src` (row pitch g.w). Returns the winner and its offset within the plane.
		// WW/WH > 0: window extents known at compile time (fully unrolled); CLIP: the window may stick out
		// of the input (round-up) and is clipped. The scan order (x fastest) and the strict compare are the
		// plain backend's (max_subsampling_layer_updater_plain.cpp:146-159).
		// MINMAX: 0 = the layer's is_min flag is read per candidate, 1 = maximum, 2 = minimum (decided once per call site)
		template <int WW, int WH, bool CLIP, int MINMAX = 0>
		__device__ __forceinline__ void scan_window(const pool_geom& g, const float * src, uint32_t oy, uint32_t ox, float& best, uint32_t& best_off)
		{
			const int win_w = WW ? WW : g.win_w, win_h = WH ? WH : g.win_h;
			const uint32_t iy0 = oy * g.sh, ix0 = ox * g.sw;
			const uint32_t off0 = iy0 * g.w + ix0;
			best = src[off0]; // the first element always seeds the result
			best_off = off0;
			#pragma unroll
			for (int ky = 0; ky < win_h; ++ky)
			{
				if (CLIP && iy0 + ky >= g.h)
					break;
				#pragma unroll
				for (int kx = 0; kx < win_w; ++kx)
				{
					if (ky == 0 && kx == 0)
						continue;
					if (CLIP && ix0 + kx >= g.w)
						break;
					const uint32_t off = off0 + ky * g.w + kx;
					const float v = src[off];
					const bool better = MINMAX == 1 ? (v > best) : (MINMAX == 2 ? (v < best) : (g.is_min ? (v < best) : (v > best)));
					if (better)
					{
						best = v;
						best_off = off;
					}
				}
			}
		}

		constexpr int kMaxGroup = 512; // planes per CTA iteration (bounds the per-plane parameter arrays)

		template <bool FUSED, int WW, int WH, bool CLIP>
		__global__ void __launch_bounds__(kThreads) pool_fwd_staged_kernel(const pool_fwd_params p)
		{
			extern __shared__ float s_z[];
			__shared__ float s_mult[FUSED ? kMaxGroup : 1];
			__shared__ float s_add[FUSED ? kMaxGroup : 1];
			const pool_geom& g = p.g;
			const int64_t ngroups = (p.planes + p.group - 1) / p.group;
			const bool has_bn = FUSED && p.gamma != nullptr;
			const bool has_res = FUSED && p.res != nullptr;
			for (int64_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x)
			{
				const int64_t plane0 = grp * p.group;
				const uint32_t np = (uint32_t)((p.planes - plane0 < p.group) ? (p.planes - plane0) : p.group);
				const uint32_t count = np * g.hw;
				const int64_t base = plane0 * g.hw;
				const float * x = p.x + base;
				if (has_bn)
				{
					// batch-norm scale/shift of each plane of the group (batch_norm_layer_tester_plain.cpp:60-61)
					const uint32_t ch0 = (uint32_t)(plane0 - int64_t(g.d_c.div((uint32_t)plane0)) * g.c);
					for (uint32_t lp = threadIdx.x; lp < np; lp += kThreads)
					{
						uint32_t channel = ch0 + lp;
						channel -= g.d_c.div(channel) * g.c;
						const float mult = __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel));
						s_mult[lp] = mult;
						s_add[lp] = __fsub_rn(__ldg(p.beta + channel), __fmul_rn(mult, __ldg(p.mean + channel)));
					}
					__syncthreads();
				}
				auto fused = [&](float v, float r, float mult, float add) -> float
				{
					float t = v;
					if (has_bn)
						t = __fadd_rn(__fmul_rn(v, mult), add);
					if (has_res)
						t = __fadd_rn(__fadd_rn(0.0F, t), r); // add layer, alpha = 1: (0 + bn) + residual
					return t >= 0.0F ? t : __fmul_rn(t, p.slope);
				};

				// phase 1: stream the group in, apply the fused per-element chain, keep it in shared memory
				if (p.vec_ok)
				{
					const uint32_t nvec = count >> 2;
					const float4 * x4 = reinterpret_cast<const float4 *>(x);
					const float4 * r4 = has_res ? reinterpret_cast<const float4 *>(p.res + base) : nullptr;
					float4 * z4 = FUSED ? reinterpret_cast<float4 *>(p.z + base) : nullptr;
					float4 * s4 = reinterpret_cast<float4 *>(s_z);
					const bool plane_per_vec = (g.hw & 3) == 0;
					constexpr int kInFlight = 2;   // independent 128-bit loads per thread and tensor before any is consumed (4: no gain)
					for (uint32_t v0 = threadIdx.x; v0 < nvec; v0 += kThreads * kInFlight)
					{
						float4 a[kInFlight], r[kInFlight];
						#pragma unroll
						for (int u = 0; u < kInFlight; ++u)
						{
							const uint32_t v = v0 + u * kThreads;
							r[u] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
							if (v < nvec)
							{
								a[u] = ld_stream(x4 + v);
								if (has_res)
									r[u] = ld_stream(r4 + v);
							}
						}
						#pragma unroll
						for (int u = 0; u < kInFlight; ++u)
						{
							const uint32_t v = v0 + u * kThreads;
							if (v < nvec)
							{
								float4 o = a[u];
								if (FUSED)
								{
									if (plane_per_vec)
									{
										const uint32_t lp = g.d_hw.div(v << 2);
										const float mult = has_bn ? s_mult[lp] : 1.0F, add = has_bn ? s_add[lp] : 0.0F;
										o.x = fused(a[u].x, r[u].x, mult, add); o.y = fused(a[u].y, r[u].y, mult, add);
										o.z = fused(a[u].z, r[u].z, mult, add); o.w = fused(a[u].w, r[u].w, mult, add);
									}
									else
									{
										// H*W not a multiple of 4: the vector may straddle one plane boundary
										const uint32_t lp0 = g.d_hw.div(v << 2);
										const uint32_t left = (lp0 + 1) * g.hw - (v << 2); // elements of this vector in plane lp0 (>= 1)
										const uint32_t lp1 = left >= 4 ? lp0 : lp0 + 1;
										const float m0 = has_bn ? s_mult[lp0] : 1.0F, a0 = has_bn ? s_add[lp0] : 0.0F;
										const float m1 = has_bn ? s_mult[lp1] : 1.0F, a1 = has_bn ? s_add[lp1] : 0.0F;
										o.x = fused(a[u].x, r[u].x, m0, a0);
										o.y = fused(a[u].y, r[u].y, left > 1 ? m0 : m1, left > 1 ? a0 : a1);
										o.z = fused(a[u].z, r[u].z, left > 2 ? m0 : m1, left > 2 ? a0 : a1);
										o.w = fused(a[u].w, r[u].w, left > 3 ? m0 : m1, left > 3 ? a0 : a1);
									}
									st_stream(z4 + v, o);
								}
								s4[v] = o;
							}
						}
					}
					for (uint32_t e = (nvec << 2) + threadIdx.x; e < count; e += kThreads)
					{
						float a = x[e];
						if (FUSED)
						{
							const uint32_t lp = g.d_hw.div(e);
							a = fused(a, has_res ? p.res[base + e] : 0.0F, has_bn ? s_mult[lp] : 1.0F, has_bn ? s_add[lp] : 0.0F);
							p.z[base + e] = a;
						}
						s_z[e] = a;
					}
				}
				else
				{
					for (uint32_t e = threadIdx.x; e < count; e += kThreads)
					{
						float a = ld_stream(x + e);
						if (FUSED)
						{
							const uint32_t lp = g.d_hw.div(e);
							a = fused(a, has_res ? ld_stream(p.res + base + e) : 0.0F, has_bn ? s_mult[lp] : 1.0F, has_bn ? s_add[lp] : 0.0F);
							st_stream(p.z + base + e, a);
						}
						s_z[e] = a;
					}
				}
				__syncthreads();

				// phase 2: windows from shared memory
				const uint32_t nout = np * g.ohw;
				const int64_t obase = plane0 * g.ohw;
				const bool is_min = g.is_min != 0;   // uniform: the comparison is chosen once, not per candidate
				for (uint32_t o = threadIdx.x; o < nout; o += kThreads)
				{
					const uint32_t lp = g.d_ohw.div(o);
					const uint32_t rem = o - lp * g.ohw;
					const uint32_t oy = g.d_ow.div(rem);
					const uint32_t ox = rem - oy * g.ow;
					float best;
					uint32_t off;
					if (is_min)
						scan_window<WW, WH, CLIP, 2>(g, s_z + lp * g.hw, oy, ox, best, off);
					else
						scan_window<WW, WH, CLIP, 1>(g, s_z + lp * g.hw, oy, ox, best, off);
					st_stream(p.pooled + obase + o, best);
					if (p.argmax)
						p.argmax[obase + o] = (uint32_t)(base + int64_t(lp) * g.hw + off);
				}
				__syncthreads();
			}
		}

		// Fallback for planes that do not fit shared memory: one thread per output element, from global.
		__global__ void __launch_bounds__(kThreads) pool_fwd_direct_kernel(float * pooled, uint32_t * argmax, const float * x, pool_geom g, int64_t planes)
		{
			const int64_t total = planes * g.ohw;
			const int64_t stride = int64_t(gridDim.x) * kThreads;
			for (int64_t o = int64_t(blockIdx.x) * kThreads + threadIdx.x; o < total; o += stride)
			{
				const int64_t plane = o / g.ohw;
				const uint32_t rem = (uint32_t)(o - plane * g.ohw);
				const uint32_t oy = g.d_ow.div(rem);
				const uint32_t ox = rem - oy * g.ow;
				float best;
				uint32_t off;
				scan_window<0, 0, true>(g, x + plane * g.hw, oy, ox, best, off);
				pooled[o] = best;
				if (argmax)
					argmax[o] = (uint32_t)(plane * g.hw + off);
			}
		}

		struct pool_bwd_params
		{
			pool_geom g;
			float * dx;            // may be null (fused)
			float * dres;          // fused only, may be null
			const float * dpooled;
			const uint32_t * argmax;
			const float * z;       // fused only
			const float * gamma;   // fused: null -> dx = ds
			const float * invsigma;
			float slope;
			int64_t planes;
			int group;
			int vec_ok;
			int add;               // stand-alone only
			int row4_vec;          // 3x3/2 fast path: rows are whole float4s (W % 4 == 0, aligned buffers)
			fastdiv d_cpr, d_hcpr; // 3x3/2 fast path with ragged rows: chunks per row, chunks per plane
		};

		// Gradient reaching input element (iy, ix) of a plane whose pooled gradients / argmax start at
		// dyp / idx; abs_off is the element's absolute offset as the argmax stores it. Windows are visited in
		// ascending output index. WW/WH/SW/SH > 0: compile-time window and stride (divisions become shifts
		// and the candidate loops unroll to ceil(WH/SH) x ceil(WW/SW) predicated steps).
		template <int WW, int WH, int SW, int SH>
		__device__ __forceinline__ float gather_element(const pool_geom& g, const float * dyp, const uint32_t * idx, uint32_t iy, uint32_t ix, uint32_t abs_off, float seed)
		{
			const uint32_t win_w = WW ? WW : g.win_w, win_h = WH ? WH : g.win_h;
			const uint32_t oy_lo = iy < win_h ? 0u : (SH ? (iy - win_h) / (SH ? SH : 1) : g.d_sh.div(iy - win_h)) + 1u;
			uint32_t oy_hi = SH ? iy / (SH ? SH : 1) : g.d_sh.div(iy);
			if (oy_hi > g.oh - 1)
				oy_hi = g.oh - 1;
			const uint32_t ox_lo = ix < win_w ? 0u : (SW ? (ix - win_w) / (SW ? SW : 1) : g.d_sw.div(ix - win_w)) + 1u;
			uint32_t ox_hi = SW ? ix / (SW ? SW : 1) : g.d_sw.div(ix);
			if (ox_hi > g.ow - 1)
				ox_hi = g.ow - 1;
			float sum = seed;
			if (WW && WH && SW && SH)
			{
				constexpr int NY = (WH + (SH ? SH : 1) - 1) / (SH ? SH : 1), NX = (WW + (SW ? SW : 1) - 1) / (SW ? SW : 1);
				#pragma unroll
				for (int a = 0; a < NY; ++a)
				{
					#pragma unroll
					for (int b = 0; b < NX; ++b)
					{
						const uint32_t oy = oy_lo + a, ox = ox_lo + b;
						if (oy <= oy_hi && ox <= ox_hi)
						{
							const uint32_t o = oy * g.ow + ox;
							if (idx[o] == abs_off)
								sum = __fadd_rn(sum, dyp[o]);
						}
					}
				}
			}
			else
			{
				for (uint32_t oy = oy_lo; oy <= oy_hi; ++oy)
					for (uint32_t ox = ox_lo; ox <= ox_hi; ++ox)
					{
						const uint32_t o = oy * g.ow + ox;
						if (idx[o] == abs_off)
							sum = __fadd_rn(sum, dyp[o]);
					}
			}
			return sum;
		}

		// 3x3 windows, stride 2, four consecutive elements of one input row (W % 4 == 0). The four elements
		// share their candidate windows: rows {oy_lo..oy_hi} (at most two) and columns {k-1, k, k+1} with
		// k = ix0/2, so a vector needs 6 (argmax, gradient) pairs instead of 16. Within a row the columns
		// are visited in ascending order, rows in ascending order: ascending output index per element.
		__device__ __forceinline__ void gather_row4_3x3s2(const pool_geom& g, const float * dyp, const uint32_t * idp, uint32_t iy, uint32_t ix0,
			uint32_t abs0, float (&acc)[4])
		{
			const uint32_t r0 = iy < 3 ? 0u : ((iy - 3) >> 1) + 1u;
			const uint32_t r1 = min(iy >> 1, g.oh - 1);
			const uint32_t k = ix0 >> 1;
			const bool c0 = k >= 1 && k - 1 <= g.ow - 1, c1 = k <= g.ow - 1, c2 = k + 1 <= g.ow - 1;
			#pragma unroll
			for (int a = 0; a < 2; ++a)
			{
				const uint32_t oy = r0 + a;
				if (oy <= r1)
				{
					const uint32_t row = oy * g.ow + k;
					if (c0)
					{
						const uint32_t i = idp[row - 1];
						const float d = dyp[row - 1];
						if (i == abs0) acc[0] = __fadd_rn(acc[0], d);
					}
					if (c1)
					{
						const uint32_t i = idp[row];
						const float d = dyp[row];
						if (i == abs0) acc[0] = __fadd_rn(acc[0], d);
						if (i == abs0 + 1) acc[1] = __fadd_rn(acc[1], d);
						if (i == abs0 + 2) acc[2] = __fadd_rn(acc[2], d);
					}
					if (c2)
					{
						const uint32_t i = idp[row + 1];
						const float d = dyp[row + 1];
						if (i == abs0 + 2) acc[2] = __fadd_rn(acc[2], d);
						if (i == abs0 + 3) acc[3] = __fadd_rn(acc[3], d);
					}
				}
			}
		}

		// 2x2 windows, stride 2, four consecutive elements of one input row: windows do not overlap, the four elements
		// belong to the two windows {k, k + 1} of output row iy / 2, k = ix0 / 2 - two (argmax, gradient) pairs per vector
		__device__ __forceinline__ void gather_row4_2x2s2(const pool_geom& g, const float * dyp, const uint32_t * idp, uint32_t iy, uint32_t ix0,
			uint32_t abs0, float (&acc)[4])
		{
			const uint32_t oy = iy >> 1;
			if (oy > g.oh - 1)
				return;
			const uint32_t k = ix0 >> 1;
			const uint32_t row = oy * g.ow + k;
			if (k <= g.ow - 1)
			{
				const uint32_t i = idp[row];
				const float d = dyp[row];
				if (i == abs0) acc[0] = __fadd_rn(acc[0], d);
				if (i == abs0 + 1) acc[1] = __fadd_rn(acc[1], d);
			}
			if (k + 1 <= g.ow - 1)
			{
				const uint32_t i = idp[row + 1];
				const float d = dyp[row + 1];
				if (i == abs0 + 2) acc[2] = __fadd_rn(acc[2], d);
				if (i == abs0 + 3) acc[3] = __fadd_rn(acc[3], d);
			}
		}

		template <int WW>
		__device__ __forceinline__ void gather_row4(const pool_geom& g, const float * dyp, const uint32_t * idp, uint32_t iy, uint32_t ix0,
			uint32_t abs0, float (&acc)[4])
		{
			if (WW == 2)
				gather_row4_2x2s2(g, dyp, idp, iy, ix0, abs0, acc);
			else
				gather_row4_3x3s2(g, dyp, idp, iy, ix0, abs0, acc);
		}

		template <bool FUSED, int WW, int WH, int SW, int SH, bool ROW4 = false>
		__global__ void __launch_bounds__(kThreads) pool_bwd_staged_kernel(const pool_bwd_params p)
		{
			extern __shared__ float s_raw[];
			const pool_geom& g = p.g;
			const int64_t ngroups = (p.planes + p.group - 1) / p.group;
			float * s_dy = s_raw;
			uint32_t * s_idx = reinterpret_cast<uint32_t *>(s_raw + size_t(p.group) * g.ohw);
			float * s_dz = s_raw + ((size_t(p.group) * g.ohw * 2 + 3) & ~size_t(3)); // ragged-row fused path only
			float * s_mult = s_dz + ((size_t(p.group) * g.hw + 3) & ~size_t(3));       // same path: gamma*invsigma per plane
			for (int64_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x)
			{
				const int64_t plane0 = grp * p.group;
				const uint32_t np = (uint32_t)((p.planes - plane0 < p.group) ? (p.planes - plane0) : p.group);
				const uint32_t nout = np * g.ohw;
				const int64_t obase = plane0 * g.ohw;
				for (uint32_t o = threadIdx.x; o < nout; o += kThreads)
				{
					s_dy[o] = ld_stream(p.dpooled + obase + o);
					s_idx[o] = __ldcs(p.argmax + obase + o);
				}
				const uint32_t ch0 = (uint32_t)(plane0 - int64_t(g.d_c.div((uint32_t)plane0)) * g.c);
				if (FUSED && ROW4 && !p.row4_vec)
					for (uint32_t lp = threadIdx.x; lp < np; lp += kThreads)
					{
						uint32_t channel = ch0 + lp;
						channel -= g.d_c.div(channel) * g.c;
						s_mult[lp] = p.gamma ? __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel)) : 1.0F;
					}
				__syncthreads();

				const uint32_t count = np * g.hw;
				const int64_t base = plane0 * g.hw;
				auto element = [&](uint32_t e, float zval, float seed, float& out_dx, float& out_dres)
				{
					const uint32_t lp = g.d_hw.div(e);
					const uint32_t rem = e - lp * g.hw;
					const uint32_t iy = g.d_w.div(rem);
					const uint32_t ix = rem - iy * g.w;
					const float dz = gather_element<WW, WH, SW, SH>(g, s_dy + lp * g.ohw, s_idx + lp * g.ohw, iy, ix, (uint32_t)(base + e), seed);
					if (FUSED)
					{
						// ReLU gate from the sign bit of z (negative pre-activations were multiplied by a
						// slope >= 0, so their sign bit is set, -0.0 included); add layer backward with
						// alpha 1 is the identity; frozen batch norm scales by gamma*invsigma.
						const float ds = (__float_as_uint(zval) >> 31) ? __fmul_rn(dz, p.slope) : dz;
						out_dres = ds;
						if (p.gamma)
						{
							uint32_t channel = ch0 + lp;
							channel -= g.d_c.div(channel) * g.c;
							out_dx = __fmul_rn(ds, __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel)));
						}
						else
							out_dx = ds;
					}
					else
						out_dx = dz;
				};

				if (ROW4 && !p.row4_vec)
				{
					// rows that are not a multiple of four elements (14x14, 7x7): the same four-element row
					// chunks, with scalar accesses and the last chunk of a row cut short
					const uint32_t cpr = (g.w + 3) >> 2;           // chunks per row
					const uint32_t nchunks = np * g.h * cpr;
					for (uint32_t q = threadIdx.x; q < nchunks; q += kThreads)
					{
						const uint32_t lp = p.d_hcpr.div(q);
						const uint32_t rem = q - lp * (g.h * cpr);
						const uint32_t iy = p.d_cpr.div(rem);
						const uint32_t ix0 = (rem - iy * cpr) << 2;
						const uint32_t e0 = lp * g.hw + iy * g.w + ix0;
						const uint32_t nvalid = min(4u, g.w - ix0);
						float acc[4] = {0.0F, 0.0F, 0.0F, 0.0F};
						if (!FUSED && p.add)
						{
							#pragma unroll
							for (int k = 0; k < 4; ++k)
								if ((uint32_t)k < nvalid)
									acc[k] = p.dx[base + e0 + k];
						}
						gather_row4<WW>(g, s_dy + lp * g.ohw, s_idx + lp * g.ohw, iy, ix0, (uint32_t)(base + e0), acc);
						#pragma unroll
						for (int k = 0; k < 4; ++k)
							if ((uint32_t)k < nvalid)
							{
								// (staging the stand-alone result too and storing it with 128-bit stores was measured slower:
								// 14x14 81 -> 100 us)
								if (FUSED)
									s_dz[e0 + k] = acc[k]; // gathered gradient of the group, consumed with coalesced accesses below
								else
									p.dx[base + e0 + k] = acc[k];
							}
					}
					if (FUSED)
					{
						__syncthreads();
						// the batch-norm factor of a plane comes from shared memory; a vector of four elements lies in
						// one plane unless it straddles a plane boundary (H*W not a multiple of 4)
						auto finish = [&](float mult, float zval, float dz, float& odx, float& ores)
						{
							const float ds = (__float_as_uint(zval) >> 31) ? __fmul_rn(dz, p.slope) : dz;
							ores = ds;
							odx = p.gamma ? __fmul_rn(ds, mult) : ds;
						};
						const uint32_t nvec = p.vec_ok ? (count >> 2) : 0;
						for (uint32_t v = threadIdx.x; v < nvec; v += kThreads)
						{
							const float4 z4 = ld_stream(reinterpret_cast<const float4 *>(p.z + base) + v);
							const float4 d4 = reinterpret_cast<const float4 *>(s_dz)[v];
							const uint32_t lp0 = g.d_hw.div(v << 2);
							const uint32_t left = (lp0 + 1) * g.hw - (v << 2); // elements of this vector in plane lp0 (>= 1)
							const float m0 = s_mult[lp0];
							const float m1 = left >= 4 ? m0 : s_mult[lp0 + 1];
							float4 ox, orr;
							finish(m0, z4.x, d4.x, ox.x, orr.x);
							finish(left > 1 ? m0 : m1, z4.y, d4.y, ox.y, orr.y);
							finish(left > 2 ? m0 : m1, z4.z, d4.z, ox.z, orr.z);
							finish(left > 3 ? m0 : m1, z4.w, d4.w, ox.w, orr.w);
							if (p.dx)
								st_stream(reinterpret_cast<float4 *>(p.dx + base) + v, ox);
							if (p.dres)
								st_stream(reinterpret_cast<float4 *>(p.dres + base) + v, orr);
						}
						for (uint32_t e = (nvec << 2) + threadIdx.x; e < count; e += kThreads)
						{
							float odx, ores;
							finish(s_mult[g.d_hw.div(e)], p.z[base + e], s_dz[e], odx, ores);
							if (p.dx)
								p.dx[base + e] = odx;
							if (p.dres)
								p.dres[base + e] = ores;
						}
					}
				}
				else if (p.vec_ok)
				{
					const uint32_t nvec = count >> 2;
					for (uint32_t v = threadIdx.x; v < nvec; v += kThreads)
					{
						float zv[4] = {0.0F, 0.0F, 0.0F, 0.0F};
						float seed[4] = {0.0F, 0.0F, 0.0F, 0.0F};
						if (FUSED)
						{
							const float4 z4 = ld_stream(reinterpret_cast<const float4 *>(p.z + base) + v);
							zv[0] = z4.x; zv[1] = z4.y; zv[2] = z4.z; zv[3] = z4.w;
						}
						else if (p.add)
						{
							const float4 d4 = ld_stream(reinterpret_cast<const float4 *>(p.dx + base) + v);
							seed[0] = d4.x; seed[1] = d4.y; seed[2] = d4.z; seed[3] = d4.w;
						}
						float odx[4], ores[4];
						if (ROW4)
						{
							const uint32_t e0 = v << 2;
							const uint32_t lp = g.d_hw.div(e0);
							const uint32_t rem = e0 - lp * g.hw;
							const uint32_t iy = g.d_w.div(rem);
							gather_row4<WW>(g, s_dy + lp * g.ohw, s_idx + lp * g.ohw, iy, rem - iy * g.w, (uint32_t)(base + e0), seed);
							float mult = 1.0F;
							if (FUSED && p.gamma)
							{
								uint32_t channel = ch0 + lp;
								channel -= g.d_c.div(channel) * g.c;
								mult = __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel));
							}
							#pragma unroll
							for (int k = 0; k < 4; ++k)
							{
								if (FUSED)
								{
									const float ds = (__float_as_uint(zv[k]) >> 31) ? __fmul_rn(seed[k], p.slope) : seed[k];
									ores[k] = ds;
									odx[k] = p.gamma ? __fmul_rn(ds, mult) : ds;
								}
								else
									odx[k] = seed[k];
							}
						}
						else
						{
							#pragma unroll
							for (int k = 0; k < 4; ++k)
								element((v << 2) + k, zv[k], seed[k], odx[k], ores[k]);
						}
						if (p.dx)
							st_stream(reinterpret_cast<float4 *>(p.dx + base) + v, make_float4(odx[0], odx[1], odx[2], odx[3]));
						if (FUSED && p.dres)
							st_stream(reinterpret_cast<float4 *>(p.dres + base) + v, make_float4(ores[0], ores[1], ores[2], ores[3]));
					}
					for (uint32_t e = (nvec << 2) + threadIdx.x; e < count; e += kThreads)
					{
						float odx, ores;
						element(e, FUSED ? p.z[base + e] : 0.0F, (!FUSED && p.add) ? p.dx[base + e] : 0.0F, odx, ores);
						if (p.dx)
							p.dx[base + e] = odx;
						if (FUSED && p.dres)
							p.dres[base + e] = ores;
					}
				}
				else
				{
					for (uint32_t e = threadIdx.x; e < count; e += kThreads)
					{
						float odx, ores;
						element(e, FUSED ? p.z[base + e] : 0.0F, (!FUSED && p.add) ? p.dx[base + e] : 0.0F, odx, ores);
						if (p.dx)
							p.dx[base + e] = odx;
						if (FUSED && p.dres)
							p.dres[base + e] = ores;
					}
				}
				__syncthreads();
			}
		}

		// Fallback gather from global memory, one thread per input element.
		template <bool FUSED>
		__global__ void __launch_bounds__(kThreads) pool_bwd_direct_kernel(const pool_bwd_params p)
		{
			const pool_geom& g = p.g;
			const int64_t total = p.planes * g.hw;
			const int64_t stride = int64_t(gridDim.x) * kThreads;
			for (int64_t e = int64_t(blockIdx.x) * kThreads + threadIdx.x; e < total; e += stride)
			{
				const int64_t plane = e / g.hw;
				const uint32_t rem = (uint32_t)(e - plane * g.hw);
				const uint32_t iy = g.d_w.div(rem);
				const uint32_t ix = rem - iy * g.w;
				const float seed = (!FUSED && p.add) ? p.dx[e] : 0.0F;
				const float dz = gather_element<0, 0, 0, 0>(g, p.dpooled + plane * g.ohw, p.argmax + plane * g.ohw, iy, ix, (uint32_t)e, seed);
				if (FUSED)
				{
					const float ds = (__float_as_uint(p.z[e]) >> 31) ? __fmul_rn(dz, p.slope) : dz;
					if (p.dres)
						p.dres[e] = ds;
					if (p.dx)
					{
						const uint32_t channel = (uint32_t)(plane % g.c);
						p.dx[e] = p.gamma ? __fmul_rn(ds, __fmul_rn(__ldg(p.gamma + channel), __ldg(p.invsigma + channel))) : ds;
					}
				}
				else
					p.dx[e] = dz;
			}
		}

		// grid size in units of one resident wave of CTAs (tuning aid: NNF_POOL_WAVES)
		int pool_waves()
		{
			return tune().pool_waves > 0 ? tune().pool_waves : 4;
		}

		int make_geom(pool_geom& g, const char * who, int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool)
		{
			if (!pool)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: pool descriptor is null", who);
			if (n < 0 || c <= 0 || h <= 0 || w <= 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: bad extents n=%lld c=%lld h=%lld w=%lld", who, (long long)n, (long long)c, (long long)h, (long long)w);
			if (pool->win_w < 1 || pool->win_h < 1 || pool->stride_w < 1 || pool->stride_h < 1)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: window and stride must be >= 1", who);
			if (h * w > kMaxElemsPerLaunch || c > 0x7fffffff)
				return set_error(NNF_ERR_UNSUPPORTED, "%s: plane too large", who);
			const int64_t ow = nnf_pool_out_size(w, pool->win_w, pool->stride_w, pool->round_up_w);
			const int64_t oh = nnf_pool_out_size(h, pool->win_h, pool->stride_h, pool->round_up_h);
			if (ow <= 0 || oh <= 0)
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: input %lldx%lld produces an empty output", who, (long long)w, (long long)h); // max_subsampling_layer.cpp:129-130
			g.c = (uint32_t)c; g.h = (uint32_t)h; g.w = (uint32_t)w; g.hw = (uint32_t)(h * w);
			g.oh = (uint32_t)oh; g.ow = (uint32_t)ow; g.ohw = (uint32_t)(oh * ow);
			g.win_w = pool->win_w; g.win_h = pool->win_h; g.sw = pool->stride_w; g.sh = pool->stride_h;
			g.is_min = pool->is_min ? 1 : 0;
			g.d_w = fastdiv(g.w); g.d_hw = fastdiv(g.hw); g.d_ow = fastdiv(g.ow); g.d_ohw = fastdiv(g.ohw);
			g.d_sw = fastdiv((uint32_t)g.sw); g.d_sh = fastdiv((uint32_t)g.sh); g.d_c = fastdiv(g.c);
			return NNF_OK;
		}

		// planes per CTA iteration; 0 -> does not fit shared memory
		int choose_group(const pool_geom& g, int64_t planes, bool& vec_ok)
		{
			// measured: 32 KB groups for large planes (56x56), 16 KB for small ones (more CTAs per SM)
			const int64_t group_floats = tune().pool_group_floats > 0 ? tune().pool_group_floats : (g.hw >= 2048 ? kGroupFloats : kGroupFloats / 2);
			int64_t grp = group_floats / g.hw;
			if (grp < 1)
				grp = 1;
			if (size_t(grp) * g.hw * sizeof(float) > staging_smem_limit())
				return 0;
			if (grp >= 4 && (g.hw % 4) != 0)
				grp &= ~int64_t(3);
			// keep at least ~4 groups per SM so that the grid stays balanced
			while (grp > 4 && div_up(planes, grp) < int64_t(sm_count()) * 4)
				grp = (grp / 2) & ~int64_t(3);
			if (grp < 1)
				grp = 1;
			if (grp > kMaxGroup)
				grp = kMaxGroup;
			if (planes < 0x7fffffff && grp > planes)
				grp = planes;
			vec_ok = vec_ok && ((grp * g.hw) % 4 == 0);
			return (int)grp;
		}

		int run_pool_fwd(cudaStream_t s, bool fused, pool_fwd_params& p, int64_t n)
		{
			// only round-up makes the last window stick out of the input
			const bool need_clip = (int64_t(p.g.oh - 1) * p.g.sh + p.g.win_h > int64_t(p.g.h)) || (int64_t(p.g.ow - 1) * p.g.sw + p.g.win_w > int64_t(p.g.w));
			p.planes = n * p.g.c;
			if (p.planes == 0)
				return NNF_OK;
			if (p.planes > 0x7fffffff)
				return set_error(NNF_ERR_UNSUPPORTED, "max subsampling: more than 2^31 planes");
			if (p.argmax && p.planes * p.g.hw > int64_t(0xffffffffll))
				return set_error(NNF_ERR_UNSUPPORTED, "max subsampling: argmax offsets need n*c*h*w < 2^32");
			bool vec_ok = aligned16(p.x) && (!fused || (aligned16(p.z) && (!p.res || aligned16(p.res))));
			const int grp = choose_group(p.g, p.planes, vec_ok);
			if (grp == 0)
			{
				if (fused)
					return set_error(NNF_ERR_UNSUPPORTED, "fused max subsampling: a %ux%u plane does not fit shared memory", p.g.w, p.g.h);
				const int64_t blocks = div_up(p.planes * p.g.ohw, kThreads);
				const int grid = (int)(blocks < int64_t(sm_count()) * 8 ? blocks : int64_t(sm_count()) * 8);
				pool_fwd_direct_kernel<<<grid, kThreads, 0, s>>>(p.pooled, p.argmax, p.x, p.g, p.planes);
				return check_launch("pool_fwd_direct_kernel");
			}
			p.group = grp;
			p.vec_ok = vec_ok ? 1 : 0;
			const size_t smem = size_t(grp) * p.g.hw * sizeof(float);
			const int64_t ngroups = div_up(p.planes, grp);
			int per_sm = (int)(sm_smem_budget() / (smem + 1024));
			per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
			const int64_t cap = int64_t(sm_count()) * per_sm * pool_waves();
			const int grid = (int)(ngroups < cap ? ngroups : cap);
			const bool clip = need_clip;
			const int ww = p.g.win_w, wh = p.g.win_h;
			cudaError_t e = cudaSuccess;
#define NNF_POOL_FWD(FUSED, WW, WH, CLIP) \
			{ \
				e = cudaFuncSetAttribute(pool_fwd_staged_kernel<FUSED, WW, WH, CLIP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit()); \
				if (e == cudaSuccess) \
					pool_fwd_staged_kernel<FUSED, WW, WH, CLIP><<<grid, kThreads, smem, s>>>(p); \
			}
#define NNF_POOL_FWD_SHAPE(FUSED) \
			if (!clip && ww == 3 && wh == 3) NNF_POOL_FWD(FUSED, 3, 3, false) \
			else if (!clip && ww == 2 && wh == 2) NNF_POOL_FWD(FUSED, 2, 2, false) \
			else if (clip && ww == 3 && wh == 3) NNF_POOL_FWD(FUSED, 3, 3, true) \
			else if (clip) NNF_POOL_FWD(FUSED, 0, 0, true) \
			else NNF_POOL_FWD(FUSED, 0, 0, false)
			if (fused)
			{
				NNF_POOL_FWD_SHAPE(true)
			}
			else
			{
				NNF_POOL_FWD_SHAPE(false)
			}
#undef NNF_POOL_FWD_SHAPE
#undef NNF_POOL_FWD
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
			return check_launch("pool_fwd_staged_kernel");
		}

		int run_pool_bwd(cudaStream_t s, bool fused, pool_bwd_params& p, int64_t n)
		{
			p.planes = n * p.g.c;
			if (p.planes == 0)
				return NNF_OK;
			if (p.planes > 0x7fffffff)
				return set_error(NNF_ERR_UNSUPPORTED, "max subsampling: more than 2^31 planes");
			if (p.planes * p.g.hw > int64_t(0xffffffffll))
				return set_error(NNF_ERR_UNSUPPORTED, "max subsampling: argmax offsets need n*c*h*w < 2^32");
			bool vec_ok = (!p.dx || aligned16(p.dx)) && (!fused || (aligned16(p.z) && (!p.dres || aligned16(p.dres))));
			const int grp = choose_group(p.g, p.planes, vec_ok);
			const bool ragged_fast = fused && p.g.win_w == 3 && p.g.win_h == 3 && p.g.sw == 2 && p.g.sh == 2 && !((p.g.w & 3) == 0 && vec_ok);
			const size_t smem = (((size_t(grp) * p.g.ohw * 2 + 3) & ~size_t(3)) + (ragged_fast ? ((size_t(grp) * p.g.hw + 3) & ~size_t(3)) + size_t(grp) : 0)) * sizeof(float);
			if (grp == 0 || smem > staging_smem_limit())
			{
				const int64_t blocks = div_up(p.planes * p.g.hw, kThreads);
				const int grid = (int)(blocks < int64_t(sm_count()) * 8 ? blocks : int64_t(sm_count()) * 8);
				if (fused)
					pool_bwd_direct_kernel<true><<<grid, kThreads, 0, s>>>(p);
				else
					pool_bwd_direct_kernel<false><<<grid, kThreads, 0, s>>>(p);
				return check_launch("pool_bwd_direct_kernel");
			}
			p.group = grp;
			p.vec_ok = vec_ok ? 1 : 0;
			const int64_t ngroups = div_up(p.planes, grp);
			int per_sm = (int)(sm_smem_budget() / (smem + 1024));
			per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
			const int64_t cap = int64_t(sm_count()) * per_sm * pool_waves();
			const int grid = (int)(ngroups < cap ? ngroups : cap);
			const int ww = p.g.win_w, wh = p.g.win_h, sw = p.g.sw, sh = p.g.sh;
			cudaError_t e = cudaSuccess;
#define NNF_POOL_BWD(FUSED, WW, WH, SW, SH) \
			{ \
				e = cudaFuncSetAttribute(pool_bwd_staged_kernel<FUSED, WW, WH, SW, SH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit()); \
				if (e == cudaSuccess) \
					pool_bwd_staged_kernel<FUSED, WW, WH, SW, SH><<<grid, kThreads, smem, s>>>(p); \
			}
			p.row4_vec = ((p.g.w & 3) == 0 && p.vec_ok) ? 1 : 0;
			p.d_cpr = fastdiv((p.g.w + 3) / 4);
			p.d_hcpr = fastdiv(p.g.h * ((p.g.w + 3) / 4));
#define NNF_POOL_BWD_SHAPE(FUSED) \
			if (ww == 3 && wh == 3 && sw == 2 && sh == 2) \
			{ \
				e = cudaFuncSetAttribute(pool_bwd_staged_kernel<FUSED, 3, 3, 2, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit()); \
				if (e == cudaSuccess) \
					pool_bwd_staged_kernel<FUSED, 3, 3, 2, 2, true><<<grid, kThreads, smem, s>>>(p); \
			} \
			else if (ww == 2 && wh == 2 && sw == 2 && sh == 2 && (p.row4_vec || !FUSED)) \
			{ \
				e = cudaFuncSetAttribute(pool_bwd_staged_kernel<FUSED, 2, 2, 2, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit()); \
				if (e == cudaSuccess) \
					pool_bwd_staged_kernel<FUSED, 2, 2, 2, 2, true><<<grid, kThreads, smem, s>>>(p); \
			} \
			else if (ww == 2 && wh == 2 && sw == 2 && sh == 2) NNF_POOL_BWD(FUSED, 2, 2, 2, 2) \
			else NNF_POOL_BWD(FUSED, 0, 0, 0, 0)
			if (fused)
			{
				NNF_POOL_BWD_SHAPE(true)
			}
			else
			{
				NNF_POOL_BWD_SHAPE(false)
			}
#undef NNF_POOL_BWD_SHAPE
#undef NNF_POOL_BWD
			if (e != cudaSuccess)
				return set_error(NNF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
			return check_launch("pool_bwd_staged_kernel");
		}
	}
}

using namespace nnf;

extern "C" int64_t nnf_pool_out_size(int64_t in_size, int32_t window, int32_t stride, int32_t round_up)
{
	if (stride < 1)
		return 0;
	// max_subsampling_layer.cpp:127
	return (in_size + stride - window + (round_up ? window - 1 : 0)) / stride;
}

extern "C" int nnf_maxpool_fwd(nnf_stream_t stream, float * y, uint32_t * argmax, const float * x,
	int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool)
{
	pool_fwd_params p = {};
	int st = make_geom(p.g, "nnf_maxpool_fwd", n, c, h, w, pool);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!y || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_maxpool_fwd: null pointer");
	p.pooled = y;
	p.argmax = argmax;
	p.x = x;
	return run_pool_fwd((cudaStream_t)stream, false, p, n);
}

extern "C" int nnf_maxpool_bwd(nnf_stream_t stream, float * dx, const float * dy, const uint32_t * argmax,
	int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool, int add_to_destination)
{
	pool_bwd_params p = {};
	int st = make_geom(p.g, "nnf_maxpool_bwd", n, c, h, w, pool);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!dx || !dy || !argmax)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_maxpool_bwd: null pointer");
	p.dx = dx;
	p.dpooled = dy;
	p.argmax = argmax;
	p.add = add_to_destination ? 1 : 0;
	return run_pool_bwd((cudaStream_t)stream, false, p, n);
}

extern "C" int nnf_bn_add_relu_maxpool_fwd(nnf_stream_t stream, float * z, float * pooled, uint32_t * argmax,
	const float * x, const float * residual,
	const float * gamma, const float * beta, const float * mean, const float * invsigma,
	float relu_slope, int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool)
{
	pool_fwd_params p = {};
	int st = make_geom(p.g, "nnf_bn_add_relu_maxpool_fwd", n, c, h, w, pool);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!z || !pooled || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_maxpool_fwd: null pointer");
	if (gamma && (!beta || !mean || !invsigma))
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_maxpool_fwd: gamma given but beta/mean/invsigma missing");
	p.z = z; p.pooled = pooled; p.argmax = argmax; p.x = x; p.res = residual;
	p.gamma = gamma; p.beta = beta; p.mean = mean; p.invsigma = invsigma;
	p.slope = relu_slope;
	return run_pool_fwd((cudaStream_t)stream, true, p, n);
}

extern "C" int nnf_bn_add_relu_maxpool_bwd(nnf_stream_t stream, float * dx, float * dresidual,
	const float * dpooled, const uint32_t * argmax, const float * z,
	const float * gamma, const float * invsigma,
	float relu_slope, int64_t n, int64_t c, int64_t h, int64_t w, const nnf_pool * pool)
{
	pool_bwd_params p = {};
	int st = make_geom(p.g, "nnf_bn_add_relu_maxpool_bwd", n, c, h, w, pool);
	if (st != NNF_OK)
		return st;
	if (n == 0)
		return NNF_OK;
	if (!dpooled || !argmax || !z)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_maxpool_bwd: null pointer");
	if (!(relu_slope >= 0.0F))
		return set_error(NNF_ERR_UNSUPPORTED, "nnf_bn_add_relu_maxpool_bwd: the ReLU gate is read from the sign of z, which needs slope >= 0 (got %g)", (double)relu_slope);
	if (gamma && !invsigma)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_bn_add_relu_maxpool_bwd: gamma given but invsigma missing");
	p.dx = dx; p.dres = dresidual; p.dpooled = dpooled; p.argmax = argmax; p.z = z;
	p.gamma = gamma; p.invsigma = invsigma; p.slope = relu_slope;
	return run_pool_bwd((cudaStream_t)stream, true, p, n);
}
