// Shared device/host helpers for the nnf_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/nnf_b200.h"

namespace nnf
{
	// ---- status / error text -------------------------------------------------------------------
	int set_error(int status, const char * fmt, ...);
	int check_launch(const char * what);

	constexpr int kSmCount = 148; // B200; grids are sized in multiples of this

	// Largest element count one launch indexes with 32-bit arithmetic. Bigger tensors are split on
	// the host into several launches at entry boundaries (or flat boundaries for shapeless ops).
	constexpr int64_t kMaxElemsPerLaunch = (int64_t(1) << 31) - 1024;

	// ---- division by a launch-invariant 32-bit divisor -------------------------------------------
	// Exact for every dividend < 2^31 (Granlund-Montgomery round-up method with a 31-bit dividend:
	// magic = ceil(2^(31+l) / d) fits in 32 bits because d > 2^(l-1)).
	struct fastdiv
	{
		uint32_t d;
		uint32_t magic;
		uint32_t shift;

		fastdiv() : d(1), magic(0), shift(0) {}

		explicit fastdiv(uint32_t divisor)
		{
			d = divisor == 0 ? 1 : divisor;
			uint32_t l = 0;
			while ((uint64_t(1) << l) < d)
				++l;
			shift = 31 + l;
			magic = uint32_t(((uint64_t(1) << shift) + d - 1) / d);
			if (d == 1)
			{
				// ceil(2^31 / 1) = 2^31 fits; shift = 31
				magic = 0x80000000u;
				shift = 31;
			}
		}

		__host__ __device__ __forceinline__ uint32_t div(uint32_t n) const
		{
#ifdef __CUDA_ARCH__
			return uint32_t((uint64_t(n) * magic) >> shift);
#else
			return uint32_t((uint64_t(n) * uint64_t(magic)) >> shift);
#endif
		}
	};

	// ---- activation arithmetic (operation order of the plain backend; no FMA contraction) -------
	struct act_param
	{
		int kind;
		float p0;
		float p1;
		const float * slope;
		float p0b;  // backward-pass constants (TanH: 1/scale and steepness*scale)
		float p1b;
	};

	struct act_chain
	{
		int n;
		act_param a[NNF_MAX_ACTS];
	};

	int make_chain(act_chain& out, const nnf_act * acts, int n_acts, bool allow_prelu);

	// Where the batch-norm scale/shift come from: running statistics (mean, invsigma) for inference,
	// or per-channel {sum, sum of squares} for training (then mean/invstd are written to `saved`).
	struct bn_source
	{
		const float * gamma;    // null -> no batch norm
		const float * beta;
		const float * mean;
		const float * invsigma;
		const float * sums;
		float * saved;
		double count_total;
		float eps;
	};

	// y = acts(((0 + bn(x)) + res) * alpha), one streaming pass (nnf_elementwise.cu)
	int run_elementwise(cudaStream_t s, float * y, const float * x, const float * res, float add_alpha,
		const bn_source& bn, const act_chain& chain, int64_t n, int64_t c, int64_t hw);

	// forward of one activation; `a` = PReLU slope of this element's channel
	template <int KIND>
	__device__ __forceinline__ float act_fwd(float v, float p0, float p1, float a)
	{
		if (KIND == NNF_ACT_RELU)
			return v >= 0.0F ? v : __fmul_rn(v, p0);                 // rectified_linear_layer_tester_plain.cpp:54
		else if (KIND == NNF_ACT_PRELU)
			return __fmul_rn(v, (v >= 0.0F ? 1.0F : a));             // parametric_rectified_linear_layer_tester_plain.cpp:66
		else if (KIND == NNF_ACT_ELU)
			return v >= 0.0F ? v : __fsub_rn(expf(v), 1.0F);         // exponential_linear_layer_tester_plain.cpp:52
		else if (KIND == NNF_ACT_TANH)
		{
			// p0 = scale, p1 = steepness*2 (hyperbolic_tangent_layer_tester_plain.cpp:44-57)
			const float e = expf(__fmul_rn(v, p1));
			return __fmul_rn(__fdiv_rn(__fsub_rn(e, 1.0F), __fadd_rn(e, 1.0F)), p0);
		}
		else if (KIND == NNF_ACT_SIGMOID)
			return __fdiv_rn(1.0F, __fadd_rn(expf(-v), 1.0F));       // sigmoid_layer_tester_plain.cpp:51
		else
			return v;
	}

	__device__ __forceinline__ float act_fwd_dyn(int kind, float v, float p0, float p1, float a)
	{
		switch (kind)
		{
		case NNF_ACT_RELU: return act_fwd<NNF_ACT_RELU>(v, p0, p1, a);
		case NNF_ACT_PRELU: return act_fwd<NNF_ACT_PRELU>(v, p0, p1, a);
		case NNF_ACT_ELU: return act_fwd<NNF_ACT_ELU>(v, p0, p1, a);
		case NNF_ACT_TANH: return act_fwd<NNF_ACT_TANH>(v, p0, p1, a);
		case NNF_ACT_SIGMOID: return act_fwd<NNF_ACT_SIGMOID>(v, p0, p1, a);
		default: return v;
		}
	}

	// derivative factor; `t` is the layer input for ReLU/PReLU and the layer output for ELU/TanH/Sigmoid.
	// For TanH p0 = 1/scale, p1 = steepness*scale (hyperbolic_tangent_layer_updater_plain.cpp:87-88).
	template <int KIND>
	__device__ __forceinline__ float act_bwd(float dy, float t, float p0, float p1, float a)
	{
		if (KIND == NNF_ACT_RELU)
			return (t >= 0.0F) ? dy : __fmul_rn(dy, p0);              // rectified_linear_layer_updater_plain.cpp:92-104
		else if (KIND == NNF_ACT_PRELU)
			return __fmul_rn(dy, (t >= 0.0F ? 1.0F : a));             // parametric_rectified_linear_layer_updater_plain.cpp:117-131
		else if (KIND == NNF_ACT_ELU)
			return __fmul_rn(dy, (t >= 0.0F) ? 1.0F : __fadd_rn(t, 1.0F)); // exponential_linear_layer_updater_plain.cpp:88-100
		else if (KIND == NNF_ACT_TANH)
		{
			const float nv = __fmul_rn(t, p0);
			return __fmul_rn(dy, __fmul_rn(p1, __fsub_rn(1.0F, __fmul_rn(nv, nv))));
		}
		else if (KIND == NNF_ACT_SIGMOID)
			return __fmul_rn(dy, __fmul_rn(t, __fsub_rn(1.0F, t)));   // sigmoid_layer_updater_plain.cpp:88-100
		else
			return dy;
	}

	// ---- memory access helpers -----------------------------------------------------------------
	// Streaming (evict-first) 128-bit accesses: every tensor on this path is touched once per kernel.
	__device__ __forceinline__ float4 ld_stream(const float4 * p) { return __ldcs(p); }
	__device__ __forceinline__ void st_stream(float4 * p, float4 v) { __stcs(p, v); }
	__device__ __forceinline__ float ld_stream(const float * p) { return __ldcs(p); }
	__device__ __forceinline__ void st_stream(float * p, float v) { __stcs(p, v); }

	inline bool aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

	inline int64_t div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }
}
