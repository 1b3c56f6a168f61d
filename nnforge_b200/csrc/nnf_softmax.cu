// Channel softmax forward/backward. HBM-bound single pass wherever one (n, pixel) column fits in
// registers or shared memory: algorithmic bytes = 8 per element forward, 12 backward.
//
// Layout cases
//   hw == 1 : the C logits of an entry are contiguous  -> one warp per row, row kept in registers
//             (C <= 1024), else one CTA per row with the row staged in shared memory.
//   hw  > 1 : logits of one pixel are hw floats apart   -> one thread per pixel, consecutive lanes on
//             consecutive pixels (coalesced 128-byte rows per channel), column kept in registers
//             (C <= 32), else a shared-memory tile [C][32 pixels] per CTA.
// Arithmetic follows nnforge/plain/softmax_layer_tester_plain.cpp:65-88 (max seeded with -1e37,
// fast_exp(x - max), multiply by the rounded reciprocal of the sum) and
// nnforge/plain/softmax_layer_updater_plain.cpp:139-160; only the order of the sum over C differs
// (tree instead of ascending), which stays inside the 1e-5 relative tolerance.
#include "nnf_common.cuh"

namespace nnf
{
	namespace
	{
		constexpr float kMaxSeed = -1.0e+37F;

		__device__ __forceinline__ float warp_max(float v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
			return v;
		}

		__device__ __forceinline__ float warp_sum(float v)
		{
			#pragma unroll
			for (int o = 16; o > 0; o >>= 1)
				v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
			return v;
		}

		// std::max(a, b) as the plain backend calls it: keeps `a` unless a < b (NaN logits never win).
		__device__ __forceinline__ float ref_max(float a, float b) { return (a < b) ? b : a; }

		// ---- hw == 1, warp per row ---------------------------------------------------------------
		// PER_LANE = ceil(c / 32) exactly: only a lane's last slot can lie past the row's end, every other guard folds away
		template <int PER_LANE, bool BACKWARD>
		__global__ void __launch_bounds__(256) softmax_rows_warp_kernel(float * out, const float * in0, const float * in1, int64_t rows, int c, int add)
		{
			const int lane = threadIdx.x & 31;
			const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
			const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
			for (int64_t row = warp; row < rows; row += nwarps)
			{
				const float * a = in0 + row * c;
				float * o = out + row * c;
				float v[PER_LANE];
				if (!BACKWARD)
				{
					// all loads first, so that they are in flight together; the dependent max chain follows
					#pragma unroll
					for (int j = 0; j < PER_LANE; ++j)
					{
						const int idx = j * 32 + lane;
						v[j] = (j + 1 < PER_LANE || idx < c) ? ld_stream(a + idx) : kMaxSeed;
					}
					float m = kMaxSeed;
					#pragma unroll
					for (int j = 0; j < PER_LANE; ++j)
						m = ref_max(m, v[j]);
					m = warp_max(m);
					float s = 0.0F;
					#pragma unroll
					for (int j = 0; j < PER_LANE; ++j)
					{
						const int idx = j * 32 + lane;
						v[j] = (j + 1 < PER_LANE || idx < c) ? fast_exp(__fsub_rn(v[j], m)) : 0.0F;
						s = __fadd_rn(s, v[j]);
					}
					s = warp_sum(s);
					const float mult = __fdiv_rn(1.0F, s);
					#pragma unroll
					for (int j = 0; j < PER_LANE; ++j)
					{
						const int idx = j * 32 + lane;
						if ((j + 1 < PER_LANE || idx < c))
							st_stream(o + idx, __fmul_rn(v[j], mult));
					}
				}
				else
				{
					// in0 = dy, in1 = y
					const float * y = in1 + row * c;
					float g[PER_LANE];
					float s = 0.0F;
					#pragma unroll
					for (int j = 0; j < PER_LANE; ++j)
					{
						const int idx = j * 32 + lane;
						g[j] = (j + 1 < PER_LANE || idx < c) ? ld_stream(a + idx) : 0.0F;
						v[j] = (j + 1 < PER_LANE || idx < c) ? ld_stream(y + idx) : 0.0F;
						s = __fadd_rn(s, __fmul_rn(g[j], v[j]));
					}
					s = warp_sum(s);
					#pragma unroll
					for (int j = 0; j < PER_LANE; ++j)
					{
						const int idx = j * 32 + lane;
						if ((j + 1 < PER_LANE || idx < c))
						{
							const float r = __fmul_rn(v[j], __fsub_rn(g[j], s));
							o[idx] = add ? __fadd_rn(o[idx], r) : r;
						}
					}
				}
			}
		}

		// ---- hw == 1, warp per row, 128-bit accesses (c % 4 == 0, 16-byte aligned rows) -------------------
		// VPL float4 per lane cover rows of up to 128*VPL logits.
		template <int VPL, bool BACKWARD>
		__global__ void __launch_bounds__(256) softmax_rows_warp4_kernel(float * out, const float * in0, const float * in1, int64_t rows, int c, int add)
		{
			const int lane = threadIdx.x & 31;
			const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
			const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
			const int c4 = c >> 2;
			for (int64_t row = warp; row < rows; row += nwarps)
			{
				const float4 * a = reinterpret_cast<const float4 *>(in0 + row * c);
				float4 * o = reinterpret_cast<float4 *>(out + row * c);
				float4 v[VPL];
				if (!BACKWARD)
				{
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
					{
						const int idx = j * 32 + lane;
						v[j] = idx < c4 ? ld_stream(a + idx) : make_float4(kMaxSeed, kMaxSeed, kMaxSeed, kMaxSeed);
					}
					float m = kMaxSeed;
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
						m = ref_max(ref_max(ref_max(ref_max(m, v[j].x), v[j].y), v[j].z), v[j].w);
					m = warp_max(m);
					float s = 0.0F;
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
					{
						const int idx = j * 32 + lane;
						if (idx < c4)
						{
							v[j].x = fast_exp(__fsub_rn(v[j].x, m)); v[j].y = fast_exp(__fsub_rn(v[j].y, m));
							v[j].z = fast_exp(__fsub_rn(v[j].z, m)); v[j].w = fast_exp(__fsub_rn(v[j].w, m));
							s = __fadd_rn(s, __fadd_rn(__fadd_rn(v[j].x, v[j].y), __fadd_rn(v[j].z, v[j].w)));
						}
					}
					s = warp_sum(s);
					const float mult = __fdiv_rn(1.0F, s);
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
					{
						const int idx = j * 32 + lane;
						if (idx < c4)
							st_stream(o + idx, make_float4(__fmul_rn(v[j].x, mult), __fmul_rn(v[j].y, mult), __fmul_rn(v[j].z, mult), __fmul_rn(v[j].w, mult)));
					}
				}
				else
				{
					const float4 * y = reinterpret_cast<const float4 *>(in1 + row * c);
					float4 g[VPL];
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
					{
						const int idx = j * 32 + lane;
						g[j] = idx < c4 ? ld_stream(a + idx) : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						v[j] = idx < c4 ? ld_stream(y + idx) : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					}
					float s = 0.0F;
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
						s = __fadd_rn(s, __fadd_rn(__fadd_rn(__fmul_rn(g[j].x, v[j].x), __fmul_rn(g[j].y, v[j].y)), __fadd_rn(__fmul_rn(g[j].z, v[j].z), __fmul_rn(g[j].w, v[j].w))));
					s = warp_sum(s);
					#pragma unroll
					for (int j = 0; j < VPL; ++j)
					{
						const int idx = j * 32 + lane;
						if (idx < c4)
						{
							float4 r = make_float4(__fmul_rn(v[j].x, __fsub_rn(g[j].x, s)), __fmul_rn(v[j].y, __fsub_rn(g[j].y, s)),
								__fmul_rn(v[j].z, __fsub_rn(g[j].z, s)), __fmul_rn(v[j].w, __fsub_rn(g[j].w, s)));
							if (add)
							{
								const float4 old = o[idx];
								r = make_float4(__fadd_rn(old.x, r.x), __fadd_rn(old.y, r.y), __fadd_rn(old.z, r.z), __fadd_rn(old.w, r.w));
							}
							st_stream(o + idx, r);
						}
					}
				}
			}
		}

		__device__ __forceinline__ float block_reduce(float v, float * s_red, bool is_max)
		{
			const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
			v = is_max ? warp_max(v) : warp_sum(v);
			__syncthreads();
			if (lane == 0)
				s_red[w] = v;
			__syncthreads();
			float r = is_max ? kMaxSeed : 0.0F;
			for (int i = 0; i < nw; ++i)
				r = is_max ? fmaxf(r, s_red[i]) : __fadd_rn(r, s_red[i]);
			return r;
		}

		// ---- hw == 1, CTA per row; the row lives in shared memory when it fits, else it is re-read ----
		// THREADS: 256, or 1024 for rows of thousands of logits (one such row fills an SM's shared memory, so the CTA's
		// own warps are all the parallelism the SM has). VEC: 128-bit accesses (c % 4 == 0, 16-byte aligned rows).
		template <bool BACKWARD, bool IN_SMEM, int THREADS, bool VEC>
		__global__ void __launch_bounds__(THREADS) softmax_rows_block_kernel(float * out, const float * in0, const float * in1, int64_t rows, int c, int add)
		{
			extern __shared__ float s_row[];
			__shared__ float s_red[THREADS / 32];
			for (int64_t row = blockIdx.x; row < rows; row += gridDim.x)
			{
				const float * a = in0 + row * c;
				float * o = out + row * c;
				if (VEC)
				{
					const int c4 = c >> 2;
					const float4 * a4 = reinterpret_cast<const float4 *>(a);
					float4 * o4 = reinterpret_cast<float4 *>(o);
					float4 * s4 = reinterpret_cast<float4 *>(s_row);
					if (!BACKWARD)
					{
						float m = kMaxSeed;
						for (int i = threadIdx.x; i < c4; i += THREADS)
						{
							const float4 v = ld_stream(a4 + i);
							if (IN_SMEM)
								s4[i] = v;
							m = ref_max(ref_max(ref_max(ref_max(m, v.x), v.y), v.z), v.w);
						}
						m = block_reduce(m, s_red, true);
						float s = 0.0F;
						for (int i = threadIdx.x; i < c4; i += THREADS)
						{
							const float4 v = IN_SMEM ? s4[i] : a4[i];
							const float4 e = make_float4(fast_exp(__fsub_rn(v.x, m)), fast_exp(__fsub_rn(v.y, m)), fast_exp(__fsub_rn(v.z, m)), fast_exp(__fsub_rn(v.w, m)));
							if (IN_SMEM)
								s4[i] = e;
							s = __fadd_rn(s, __fadd_rn(__fadd_rn(e.x, e.y), __fadd_rn(e.z, e.w)));
						}
						s = block_reduce(s, s_red, false);
						const float mult = __fdiv_rn(1.0F, s);
						for (int i = threadIdx.x; i < c4; i += THREADS)
						{
							float4 e;
							if (IN_SMEM)
								e = s4[i];
							else
							{
								const float4 v = a4[i];
								e = make_float4(fast_exp(__fsub_rn(v.x, m)), fast_exp(__fsub_rn(v.y, m)), fast_exp(__fsub_rn(v.z, m)), fast_exp(__fsub_rn(v.w, m)));
							}
							st_stream(o4 + i, make_float4(__fmul_rn(e.x, mult), __fmul_rn(e.y, mult), __fmul_rn(e.z, mult), __fmul_rn(e.w, mult)));
						}
					}
					else
					{
						// in0 = dy, in1 = y; both stay in shared memory for the second pass when they fit
						const float4 * y4 = reinterpret_cast<const float4 *>(in1 + row * c);
						float4 * sy4 = s4 + c4;
						float s = 0.0F;
						for (int i = threadIdx.x; i < c4; i += THREADS)
						{
							const float4 g = ld_stream(a4 + i), y = ld_stream(y4 + i);
							if (IN_SMEM)
							{
								s4[i] = g;
								sy4[i] = y;
							}
							s = __fadd_rn(s, __fadd_rn(__fadd_rn(__fmul_rn(g.x, y.x), __fmul_rn(g.y, y.y)), __fadd_rn(__fmul_rn(g.z, y.z), __fmul_rn(g.w, y.w))));
						}
						s = block_reduce(s, s_red, false);
						for (int i = threadIdx.x; i < c4; i += THREADS)
						{
							const float4 g = IN_SMEM ? s4[i] : a4[i], y = IN_SMEM ? sy4[i] : y4[i];
							float4 r = make_float4(__fmul_rn(y.x, __fsub_rn(g.x, s)), __fmul_rn(y.y, __fsub_rn(g.y, s)), __fmul_rn(y.z, __fsub_rn(g.z, s)), __fmul_rn(y.w, __fsub_rn(g.w, s)));
							if (add)
							{
								const float4 old = o4[i];
								r = make_float4(__fadd_rn(old.x, r.x), __fadd_rn(old.y, r.y), __fadd_rn(old.z, r.z), __fadd_rn(old.w, r.w));
							}
							st_stream(o4 + i, r);
						}
					}
				}
				else if (!BACKWARD)
				{
					float m = kMaxSeed;
					for (int i = threadIdx.x; i < c; i += THREADS)
					{
						const float v = a[i];
						if (IN_SMEM)
							s_row[i] = v;
						m = ref_max(m, v);
					}
					m = block_reduce(m, s_red, true);
					float s = 0.0F;
					for (int i = threadIdx.x; i < c; i += THREADS)
					{
						const float e = fast_exp(__fsub_rn(IN_SMEM ? s_row[i] : a[i], m));
						if (IN_SMEM)
							s_row[i] = e;
						s = __fadd_rn(s, e);
					}
					s = block_reduce(s, s_red, false);
					const float mult = __fdiv_rn(1.0F, s);
					for (int i = threadIdx.x; i < c; i += THREADS)
					{
						const float e = IN_SMEM ? s_row[i] : fast_exp(__fsub_rn(a[i], m));
						o[i] = __fmul_rn(e, mult);
					}
				}
				else
				{
					const float * y = in1 + row * c;
					float * s_y = s_row + c;
					float s = 0.0F;
					for (int i = threadIdx.x; i < c; i += THREADS)
					{
						const float g = a[i], yv = y[i];
						if (IN_SMEM)
						{
							s_row[i] = g;
							s_y[i] = yv;
						}
						s = __fadd_rn(s, __fmul_rn(g, yv));
					}
					s = block_reduce(s, s_red, false);
					for (int i = threadIdx.x; i < c; i += THREADS)
					{
						const float g = IN_SMEM ? s_row[i] : a[i], yv = IN_SMEM ? s_y[i] : y[i];
						const float r = __fmul_rn(yv, __fsub_rn(g, s));
						o[i] = add ? __fadd_rn(o[i], r) : r;
					}
				}
				__syncthreads();
			}
		}

		// ---- hw > 1, thread per pixel, column in registers ------------------------------------------
		// One instantiation per column length (CMAX = C): the guards of the unrolled loops fold away at compile time
		template <int CMAX, bool BACKWARD>
		__global__ void __launch_bounds__(256, BACKWARD ? 2 : 4) softmax_pixels_reg_kernel(float * out, const float * in0, const float * in1, int64_t pixels, uint32_t hw, fastdiv hwdiv, int add)
		{
			constexpr int c = CMAX;
			const int64_t stride = int64_t(gridDim.x) * blockDim.x;
			for (int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < pixels; p += stride)
			{
				// pixels < 2^31 per launch: entry = p / hw
				const uint32_t entry = hwdiv.div((uint32_t)p);
				const uint32_t pix = (uint32_t)p - entry * hw;
				const int64_t base = int64_t(entry) * c * hw + pix;
				float v[CMAX];
				if (!BACKWARD)
				{
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
						v[f] = (f < c) ? ld_stream(in0 + base + int64_t(f) * hw) : kMaxSeed;
					float m = kMaxSeed;
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
						m = ref_max(m, v[f]);
					float s = 0.0F;
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
					{
						if (f < c)
						{
							v[f] = fast_exp(__fsub_rn(v[f], m));
							s = __fadd_rn(s, v[f]); // ascending c: same order as the plain backend
						}
					}
					const float mult = __fdiv_rn(1.0F, s);
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
						if (f < c)
							out[base + int64_t(f) * hw] = __fmul_rn(v[f], mult);
				}
				else
				{
					float g[CMAX];
					float s = 0.0F;
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
					{
						if (f < c)
						{
							g[f] = ld_stream(in0 + base + int64_t(f) * hw);
							v[f] = ld_stream(in1 + base + int64_t(f) * hw);
						}
					}
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
						if (f < c)
							s = __fadd_rn(s, __fmul_rn(g[f], v[f]));
					#pragma unroll
					for (int f = 0; f < CMAX; ++f)
					{
						if (f < c)
						{
							const float r = __fmul_rn(v[f], __fsub_rn(g[f], s));
							float * o = out + base + int64_t(f) * hw;
							*o = add ? __fadd_rn(*o, r) : r;
						}
					}
				}
			}
		}

		// ---- hw > 1, 33 to 160 channels, planes of whole float4s: a CTA takes 128 neighbouring pixels (a float4 per lane), its
		// WARPS warps share the channels (warp w: channels w, w + WARPS, ...); forward every value stays in registers between the
		// load and the store; maxima and sums cross the warps through shared memory. One pass over DRAM, 512-byte rows ----
		template <int CPW, int WARPS, bool BACKWARD>
		__global__ void __launch_bounds__(WARPS * 32, 2) softmax_pixels_wide_kernel(float * out, const float * in0, const float * in1, int64_t quads, uint32_t hw4, fastdiv hw4div, int c, int add)
		{
			__shared__ float4 s_red[WARPS][32];
			const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
			const int64_t ntiles = (quads + 31) / 32;
			const float4 * in4 = reinterpret_cast<const float4 *>(in0);
			const float4 * y4 = reinterpret_cast<const float4 *>(in1);
			float4 * out4 = reinterpret_cast<float4 *>(out);
			for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x)
			{
				const int64_t q = t * 32 + lane;
				const bool valid = q < quads;
				const uint32_t entry = valid ? hw4div.div((uint32_t)q) : 0;
				const uint32_t pq = valid ? (uint32_t)q - entry * hw4 : 0;
				const int64_t base = int64_t(entry) * c * hw4 + pq;   // in float4s; one channel further = hw4
				if (!BACKWARD)
				{
					float4 v[CPW];
					#pragma unroll
					for (int k = 0; k < CPW; ++k)
					{
						const int f = w + k * WARPS;
						v[k] = (valid && f < c) ? ld_stream(in4 + base + int64_t(f) * hw4) : make_float4(kMaxSeed, kMaxSeed, kMaxSeed, kMaxSeed);
					}
					float4 m = make_float4(kMaxSeed, kMaxSeed, kMaxSeed, kMaxSeed);
					#pragma unroll
					for (int k = 0; k < CPW; ++k)
					{
						m.x = ref_max(m.x, v[k].x); m.y = ref_max(m.y, v[k].y);
						m.z = ref_max(m.z, v[k].z); m.w = ref_max(m.w, v[k].w);
					}
					s_red[w][lane] = m;
					__syncthreads();
					m = make_float4(kMaxSeed, kMaxSeed, kMaxSeed, kMaxSeed);
					#pragma unroll
					for (int i = 0; i < WARPS; ++i)
					{
						const float4 r = s_red[i][lane];
						m.x = fmaxf(m.x, r.x); m.y = fmaxf(m.y, r.y); m.z = fmaxf(m.z, r.z); m.w = fmaxf(m.w, r.w);
					}
					__syncthreads();
					float4 sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					#pragma unroll
					for (int k = 0; k < CPW; ++k)
					{
						const int f = w + k * WARPS;
						if (f < c)
						{
							v[k].x = fast_exp(__fsub_rn(v[k].x, m.x)); v[k].y = fast_exp(__fsub_rn(v[k].y, m.y));
							v[k].z = fast_exp(__fsub_rn(v[k].z, m.z)); v[k].w = fast_exp(__fsub_rn(v[k].w, m.w));
							sum.x = __fadd_rn(sum.x, v[k].x); sum.y = __fadd_rn(sum.y, v[k].y);
							sum.z = __fadd_rn(sum.z, v[k].z); sum.w = __fadd_rn(sum.w, v[k].w);
						}
					}
					s_red[w][lane] = sum;
					__syncthreads();
					sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					#pragma unroll
					for (int i = 0; i < WARPS; ++i)
					{
						const float4 r = s_red[i][lane];
						sum.x = __fadd_rn(sum.x, r.x); sum.y = __fadd_rn(sum.y, r.y); sum.z = __fadd_rn(sum.z, r.z); sum.w = __fadd_rn(sum.w, r.w);
					}
					const float4 mult = make_float4(__fdiv_rn(1.0F, sum.x), __fdiv_rn(1.0F, sum.y), __fdiv_rn(1.0F, sum.z), __fdiv_rn(1.0F, sum.w));
					#pragma unroll
					for (int k = 0; k < CPW; ++k)
					{
						const int f = w + k * WARPS;
						if (valid && f < c)
							st_stream(out4 + base + int64_t(f) * hw4, make_float4(__fmul_rn(v[k].x, mult.x), __fmul_rn(v[k].y, mult.y), __fmul_rn(v[k].z, mult.z), __fmul_rn(v[k].w, mult.w)));
					}
					__syncthreads();
				}
				else
				{
					// in0 = dy, in1 = y: not held between the sum and the result but read again (the second time from L2), which
					// leaves registers for two CTAs per SM ([16,150,128,128]: 87 us; 118 us with both tensors held by one 1024-thread CTA)
					float4 sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					#pragma unroll
					for (int k = 0; k < CPW; ++k)
					{
						const int f = w + k * WARPS;
						const bool on = valid && f < c;
						const float4 g = on ? __ldg(in4 + base + int64_t(f) * hw4) : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						const float4 y = on ? __ldg(y4 + base + int64_t(f) * hw4) : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
						sum.x = __fadd_rn(sum.x, __fmul_rn(g.x, y.x)); sum.y = __fadd_rn(sum.y, __fmul_rn(g.y, y.y));
						sum.z = __fadd_rn(sum.z, __fmul_rn(g.z, y.z)); sum.w = __fadd_rn(sum.w, __fmul_rn(g.w, y.w));
					}
					s_red[w][lane] = sum;
					__syncthreads();
					sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
					#pragma unroll
					for (int i = 0; i < WARPS; ++i)
					{
						const float4 r = s_red[i][lane];
						sum.x = __fadd_rn(sum.x, r.x); sum.y = __fadd_rn(sum.y, r.y); sum.z = __fadd_rn(sum.z, r.z); sum.w = __fadd_rn(sum.w, r.w);
					}
					#pragma unroll
					for (int k = 0; k < CPW; ++k)
					{
						const int f = w + k * WARPS;
						if (valid && f < c)
						{
							const float4 g = ld_stream(in4 + base + int64_t(f) * hw4), y = ld_stream(y4 + base + int64_t(f) * hw4);
							float4 r = make_float4(__fmul_rn(y.x, __fsub_rn(g.x, sum.x)), __fmul_rn(y.y, __fsub_rn(g.y, sum.y)),
								__fmul_rn(y.z, __fsub_rn(g.z, sum.z)), __fmul_rn(y.w, __fsub_rn(g.w, sum.w)));
							float4 * o = out4 + base + int64_t(f) * hw4;
							if (add)
							{
								const float4 old = *o;
								r = make_float4(__fadd_rn(old.x, r.x), __fadd_rn(old.y, r.y), __fadd_rn(old.z, r.z), __fadd_rn(old.w, r.w));
							}
							st_stream(o, r);
						}
					}
					__syncthreads();
				}
			}
		}

		// ---- hw > 1, any C: CTA = 32 pixels x 8 channel groups, column tile staged in shared memory
		// when it fits (single HBM pass), else re-read from global/L2 --------------------------------
		template <bool BACKWARD, bool IN_SMEM>
		__global__ void __launch_bounds__(256) softmax_pixels_tile_kernel(float * out, const float * in0, const float * in1, int64_t pixels, uint32_t hw, fastdiv hwdiv, int c, int add)
		{
			extern __shared__ float s_tile[]; // [c][32] when IN_SMEM (second [c][32] for backward)
			__shared__ float s_red[8][32];
			const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
			const int64_t ntiles = (pixels + 31) / 32;
			for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x)
			{
				const int64_t p = t * 32 + lane;
				const bool valid = p < pixels;
				const uint32_t entry = valid ? hwdiv.div((uint32_t)p) : 0;
				const uint32_t pix = valid ? (uint32_t)p - entry * hw : 0;
				const int64_t base = int64_t(entry) * c * hw + pix;
				if (!BACKWARD)
				{
					float m = kMaxSeed;
					// four channels of this warp's share at a time: their loads are in flight together (ascending channel order kept)
					for (int f0 = grp; f0 < c; f0 += 32)
					{
						float v[4];
						#pragma unroll
						for (int u = 0; u < 4; ++u)
						{
							const int f = f0 + 8 * u;
							v[u] = (valid && f < c) ? ld_stream(in0 + base + int64_t(f) * hw) : 0.0F;
						}
						#pragma unroll
						for (int u = 0; u < 4; ++u)
						{
							const int f = f0 + 8 * u;
							if (f < c)
							{
								if (IN_SMEM)
									s_tile[f * 32 + lane] = v[u];
								m = ref_max(m, v[u]);
							}
						}
					}
					s_red[grp][lane] = m;
					__syncthreads();
					m = kMaxSeed;
					#pragma unroll
					for (int i = 0; i < 8; ++i)
						m = fmaxf(m, s_red[i][lane]);
					__syncthreads();
					float s = 0.0F;
					for (int f = grp; f < c; f += 8)
					{
						const float x = IN_SMEM ? s_tile[f * 32 + lane] : (valid ? in0[base + int64_t(f) * hw] : 0.0F);
						const float e = fast_exp(__fsub_rn(x, m));
						if (IN_SMEM)
							s_tile[f * 32 + lane] = e;
						s = __fadd_rn(s, e);
					}
					s_red[grp][lane] = s;
					__syncthreads();
					s = 0.0F;
					#pragma unroll
					for (int i = 0; i < 8; ++i)
						s = __fadd_rn(s, s_red[i][lane]);
					const float mult = __fdiv_rn(1.0F, s);
					if (valid)
						for (int f = grp; f < c; f += 8)
						{
							const float e = IN_SMEM ? s_tile[f * 32 + lane] : fast_exp(__fsub_rn(in0[base + int64_t(f) * hw], m));
							st_stream(out + base + int64_t(f) * hw, __fmul_rn(e, mult));
						}
					__syncthreads();
				}
				else
				{
					float * s_dy = s_tile;
					float * s_y = s_tile + size_t(c) * 32;
					float s = 0.0F;
					for (int f0 = grp; f0 < c; f0 += 32)
					{
						float g[4], y[4];
						#pragma unroll
						for (int u = 0; u < 4; ++u)
						{
							const int f = f0 + 8 * u;
							g[u] = (valid && f < c) ? ld_stream(in0 + base + int64_t(f) * hw) : 0.0F;
							y[u] = (valid && f < c) ? ld_stream(in1 + base + int64_t(f) * hw) : 0.0F;
						}
						#pragma unroll
						for (int u = 0; u < 4; ++u)
						{
							const int f = f0 + 8 * u;
							if (f < c)
							{
								if (IN_SMEM)
								{
									s_dy[f * 32 + lane] = g[u];
									s_y[f * 32 + lane] = y[u];
								}
								s = __fadd_rn(s, __fmul_rn(g[u], y[u]));
							}
						}
					}
					s_red[grp][lane] = s;
					__syncthreads();
					s = 0.0F;
					#pragma unroll
					for (int i = 0; i < 8; ++i)
						s = __fadd_rn(s, s_red[i][lane]);
					if (valid)
						for (int f = grp; f < c; f += 8)
						{
							const float g = IN_SMEM ? s_dy[f * 32 + lane] : in0[base + int64_t(f) * hw];
							const float y = IN_SMEM ? s_y[f * 32 + lane] : in1[base + int64_t(f) * hw];
							const float r = __fmul_rn(y, __fsub_rn(g, s));
							float * o = out + base + int64_t(f) * hw;
							*o = add ? __fadd_rn(*o, r) : r;
						}
					__syncthreads();
				}
			}
		}


		template <bool BACKWARD>
		int run_softmax(cudaStream_t s, float * out, const float * in0, const float * in1, int64_t n, int64_t c, int64_t hw, int add)
		{
			if (hw == 1)
			{
				const int64_t rows = n;
				if (c <= 1024)
				{
					const int64_t blocks_needed = div_up(rows, 8);
					const int grid = (int)(blocks_needed < int64_t(sm_count()) * 64 ? blocks_needed : int64_t(sm_count()) * 64);
					if ((c & 3) == 0 && aligned16(out) && aligned16(in0) && (!in1 || aligned16(in1)))
					{
						// a few hundred rows (x[256,1000]: 256 warps) are a launch-latency case: one or two warps per CTA put every
						// row on an SM of its own instead of eight rows on each of 32 SMs
						const int threads4 = rows <= int64_t(sm_count()) * 2 ? 32 : (rows <= int64_t(sm_count()) * 8 ? 64 : 256);
						const int64_t blocks4 = div_up(rows, threads4 / 32);
						const int grid4 = (int)(blocks4 < int64_t(sm_count()) * 64 ? blocks4 : int64_t(sm_count()) * 64);
#define NNF_ROWS4(VPL) softmax_rows_warp4_kernel<VPL, BACKWARD><<<grid4, threads4, 0, s>>>(out, in0, in1, rows, (int)c, add)
						if (c <= 128) NNF_ROWS4(1);
						else if (c <= 256) NNF_ROWS4(2);
						else if (c <= 512) NNF_ROWS4(4);
						else NNF_ROWS4(8);
#undef NNF_ROWS4
						return check_launch("softmax_rows_warp4_kernel");
					}
#define NNF_ROWS(PL) case PL: softmax_rows_warp_kernel<PL, BACKWARD><<<grid, 256, 0, s>>>(out, in0, in1, rows, (int)c, add); break;
					switch ((int)div_up(c, 32))
					{
					NNF_ROWS(1) NNF_ROWS(2) NNF_ROWS(3) NNF_ROWS(4) NNF_ROWS(5) NNF_ROWS(6) NNF_ROWS(7) NNF_ROWS(8)
					NNF_ROWS(9) NNF_ROWS(10) NNF_ROWS(11) NNF_ROWS(12) NNF_ROWS(13) NNF_ROWS(14) NNF_ROWS(15) NNF_ROWS(16)
					NNF_ROWS(17) NNF_ROWS(18) NNF_ROWS(19) NNF_ROWS(20) NNF_ROWS(21) NNF_ROWS(22) NNF_ROWS(23) NNF_ROWS(24)
					NNF_ROWS(25) NNF_ROWS(26) NNF_ROWS(27) NNF_ROWS(28) NNF_ROWS(29) NNF_ROWS(30) NNF_ROWS(31) NNF_ROWS(32)
					default: break;
					}
#undef NNF_ROWS
					return check_launch("softmax_rows_warp_kernel");
				}
				// rows of thousands of logits: 1024 threads per CTA, two CTAs per SM, second and third pass from L2 ([8192,32000] forward:
				// 531 us with the row staged in shared memory and one CTA per SM, 471 us without); shorter rows (backward: dy and y)
				// stay in shared memory when they fit
				const bool big = c >= 4096;
				const bool vec = (c & 3) == 0 && aligned16(out) && aligned16(in0) && (!in1 || aligned16(in1));
				const size_t smem = size_t(c) * sizeof(float) * (BACKWARD ? 2 : 1);
				const bool in_smem = smem <= staging_smem_limit() && !big;
				const int per_sm = in_smem ? (int)(staging_smem_limit() / (smem < 1024 ? 1024 : smem)) : (big ? 2 : 8);
				const int64_t cap = int64_t(sm_count()) * (per_sm < 1 ? 1 : (per_sm > (big ? 2 : 8) ? (big ? 2 : 8) : per_sm));
				const int grid = (int)(rows < cap ? rows : cap);
#define NNF_BLOCK(IN, TH, VE) \
				do { \
					if (IN) \
					{ \
						cudaError_t e = cudaFuncSetAttribute(softmax_rows_block_kernel<BACKWARD, IN, TH, VE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit()); \
						if (e != cudaSuccess) \
							return set_error(NNF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e)); \
					} \
					softmax_rows_block_kernel<BACKWARD, IN, TH, VE><<<grid, TH, IN ? smem : 0, s>>>(out, in0, in1, rows, (int)c, add); \
				} while (0)
				if (in_smem)
				{
					if (big) { if (vec) NNF_BLOCK(true, 1024, true); else NNF_BLOCK(true, 1024, false); }
					else { if (vec) NNF_BLOCK(true, 256, true); else NNF_BLOCK(true, 256, false); }
				}
				else
				{
					if (big) { if (vec) NNF_BLOCK(false, 1024, true); else NNF_BLOCK(false, 1024, false); }
					else { if (vec) NNF_BLOCK(false, 256, true); else NNF_BLOCK(false, 256, false); }
				}
#undef NNF_BLOCK
				return check_launch("softmax_rows_block_kernel");
			}

			// hw > 1: split launches so that the pixel index fits 31 bits
			if (hw > 0x7fffffff || c > 0x7fffffff)
				return set_error(NNF_ERR_UNSUPPORTED, "softmax: extent too large");
			const int64_t entries_per_launch = kMaxElemsPerLaunch / hw;
			if (entries_per_launch < 1)
				return set_error(NNF_ERR_UNSUPPORTED, "softmax: hw too large");
			for (int64_t e0 = 0; e0 < n; e0 += entries_per_launch)
			{
				const int64_t ne = (n - e0 < entries_per_launch) ? (n - e0) : entries_per_launch;
				const int64_t pixels = ne * hw;
				const int64_t off = e0 * c * hw;
				float * o = out + off;
				const float * a = in0 + off;
				const float * b = in1 ? in1 + off : nullptr;
				if (c <= 32)
				{
					const int64_t blocks_needed = div_up(pixels, 256);
					const int grid = (int)(blocks_needed < int64_t(sm_count()) * 128 ? blocks_needed : int64_t(sm_count()) * 128);
					// one instantiation per column length: no dead slots in the unrolled loops and no more registers than the
					// column needs (x[32,21,128,128] forward: 20.7 us with 32 slots for 21 elements, 16.4 us with 21)
#define NNF_EXACT(C) case C: softmax_pixels_reg_kernel<C, BACKWARD><<<grid, 256, 0, s>>>(o, a, b, pixels, (uint32_t)hw, fastdiv((uint32_t)hw), add); break;
					switch ((int)c)
					{
					NNF_EXACT(1) NNF_EXACT(2) NNF_EXACT(3) NNF_EXACT(4) NNF_EXACT(5) NNF_EXACT(6) NNF_EXACT(7) NNF_EXACT(8)
					NNF_EXACT(9) NNF_EXACT(10) NNF_EXACT(11) NNF_EXACT(12) NNF_EXACT(13) NNF_EXACT(14) NNF_EXACT(15) NNF_EXACT(16)
					NNF_EXACT(17) NNF_EXACT(18) NNF_EXACT(19) NNF_EXACT(20) NNF_EXACT(21) NNF_EXACT(22) NNF_EXACT(23) NNF_EXACT(24)
					NNF_EXACT(25) NNF_EXACT(26) NNF_EXACT(27) NNF_EXACT(28) NNF_EXACT(29) NNF_EXACT(30) NNF_EXACT(31) NNF_EXACT(32)
					default: break;
					}
#undef NNF_EXACT
					int st = check_launch("softmax_pixels_reg_kernel");
					if (st != NNF_OK)
						return st;
				}
				else if (c <= 160 && hw % 4 == 0 && aligned16(o) && aligned16(a) && (!b || aligned16(b)))
				{
					// 16 warps of up to 10 channels each; forward the values stay in registers, backward dy and y are read twice
					constexpr int kWarps = 16;
					const int cpw = (int)div_up(c, kWarps);
					const int64_t quads = pixels / 4;
					const int64_t ntiles = div_up(quads, 32);
					const int64_t cap = int64_t(sm_count()) * 4;
					const int grid = (int)(ntiles < cap ? ntiles : cap);
#define NNF_WIDE(CPW) case CPW: softmax_pixels_wide_kernel<CPW, kWarps, BACKWARD><<<grid, kWarps * 32, 0, s>>>(o, a, b, quads, (uint32_t)(hw / 4), fastdiv((uint32_t)(hw / 4)), (int)c, add); break;
					switch (cpw)   // more than 32 channels: at least three per warp
					{
					NNF_WIDE(3) NNF_WIDE(4) NNF_WIDE(5) NNF_WIDE(6) NNF_WIDE(7) NNF_WIDE(8) NNF_WIDE(9) NNF_WIDE(10)
					default: break;
					}
#undef NNF_WIDE
					int st = check_launch("softmax_pixels_wide_kernel");
					if (st != NNF_OK)
						return st;
				}
				else
				{
					const int64_t ntiles = div_up(pixels, 32);
					const size_t smem = size_t(c) * 32 * sizeof(float) * (BACKWARD ? 2 : 1);
					const bool in_smem = smem <= staging_smem_limit();
					const int per_sm = in_smem ? (int)(staging_smem_limit() / (smem < 1024 ? 1024 : smem)) : 8;
					const int64_t cap = int64_t(sm_count()) * (per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm));
					const int grid = (int)(ntiles < cap ? ntiles : cap);
					if (in_smem)
					{
						cudaError_t e = cudaFuncSetAttribute(softmax_pixels_tile_kernel<BACKWARD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staging_smem_limit());
						if (e != cudaSuccess)
							return set_error(NNF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
						softmax_pixels_tile_kernel<BACKWARD, true><<<grid, 256, smem, s>>>(o, a, b, pixels, (uint32_t)hw, fastdiv((uint32_t)hw), (int)c, add);
					}
					else
						softmax_pixels_tile_kernel<BACKWARD, false><<<grid, 256, 0, s>>>(o, a, b, pixels, (uint32_t)hw, fastdiv((uint32_t)hw), (int)c, add);
					int st = check_launch("softmax_pixels_tile_kernel");
					if (st != NNF_OK)
						return st;
				}
			}
			return NNF_OK;
		}
	}
}

using namespace nnf;

extern "C" int nnf_softmax_fwd(nnf_stream_t stream, float * y, const float * x, int64_t n, int64_t c, int64_t hw)
{
	if (n < 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_softmax_fwd: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (n == 0)
		return NNF_OK;
	if (!y || !x)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_softmax_fwd: null pointer");
	return run_softmax<false>((cudaStream_t)stream, y, x, nullptr, n, c, hw, 0);
}

extern "C" int nnf_softmax_bwd(nnf_stream_t stream, float * dx, const float * dy, const float * y, int64_t n, int64_t c, int64_t hw, int add_to_destination)
{
	if (n < 0 || c <= 0 || hw <= 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_softmax_bwd: bad extents n=%lld c=%lld hw=%lld", (long long)n, (long long)c, (long long)hw);
	if (n == 0)
		return NNF_OK;
	if (!dx || !dy || !y)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_softmax_bwd: null pointer");
	return run_softmax<true>((cudaStream_t)stream, dx, dy, y, n, c, hw, add_to_destination ? 1 : 0);
}
