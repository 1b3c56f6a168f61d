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

	// ---- what the device offers (nnforge/cuda/cuda_running_configuration.h:126-153) ---------------
	// Filled once per device from cudaDeviceGetAttribute; grids are sized in multiples of the SM count and
	// shared-memory tiles against the opt-in limit, instead of literals for one chip.
	struct running_configuration
	{
		int device_id;
		int compute_capability_major, compute_capability_minor;
		int multiprocessor_count;
		int max_threads_per_multiprocessor;
		int max_shared_memory_per_block_optin;   // bytes a kernel may ask for with cudaFuncSetAttribute
		int max_shared_memory_per_multiprocessor;
		int l2_cache_size;
		int max_registers_per_multiprocessor;
	};
	const running_configuration& running_config();   // of the calling thread's current device
	inline int sm_count() { return running_config().multiprocessor_count; }
	// Most shared memory one CTA of a staging kernel asks for (the opt-in limit less room for static data
	// and a second resident CTA's reserve: 200 KB on B200), and what all CTAs of an SM can share.
	inline size_t staging_smem_limit()
	{
		const int lim = running_config().max_shared_memory_per_block_optin;
		return size_t(lim > 64 * 1024 ? lim - 27 * 1024 : lim);
	}
	inline size_t sm_smem_budget()
	{
		const int lim = running_config().max_shared_memory_per_multiprocessor;
		return size_t(lim > 64 * 1024 ? lim - 8 * 1024 : lim);
	}

	// ---- knobs of the launch plans -----------------------------------------------------------------
	// Process-wide, set through nnf_set_tuning() (tests walk the geometries with it; nothing reads the
	// environment). Values <= 0 mean "the built-in choice".
	struct tuning
	{
		int elementwise_waves;        // grid of the streaming kernel in resident waves
		int elementwise_group_waves;  // the same for the channel-group inference kernel
		int pool_waves;               // max / average subsampling grids
		int pool_group_floats;        // floats of one staged plane group
		int channel_waves;            // training kernels with one CTA per (channel, slice)
		int group_waves;              // the same for the channel-group training kernels
		int chain_s_kb, chain_a_kb;   // single-launch training kernel: KB of one tensor per statistics / apply item
		int chain_dist;               // channels between an apply item and the statistics items it shares a step with
		int chain_chunk_mb, chain_lag;// channel-group form of that kernel: chunk size and lag in chunks
		int no_grouped;               // 1: planes that are not whole float4s take the per-channel kernels
		int apply_flat;               // 1: training apply through the flat streaming kernel
		long long peer_wait_ns;       // how long a launch waits for another rank's statistics before it gives up
	};
	tuning& tune();

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
		const float * bias;     // per-channel bias added to x before everything else (a convolution's bias), or null
	};

	// y = acts(((0 + bn(x + bias)) + res) * alpha), one streaming pass (nnf_elementwise.cu)
	int run_elementwise(cudaStream_t s, float * y, const float * x, const float * res, float add_alpha,
		const bn_source& bn, const act_chain& chain, int64_t n, int64_t c, int64_t hw);

	// ---- exp and division at "tolerance" accuracy ---------------------------------------------------
	// exp(x) = 2^(x*log2 e) on the ex2 unit: two instructions where the library expf needs ~20 (the
	// elementwise kernels are instruction-bound with it). Relative error <= 2^-22 (ex2.approx) plus
	// |x| * 6e-8 from rounding x*log2(e): below 6e-6 for every finite result and below 1e-6 for
	// |x| <= 12. Every use on this path either has x <= 0 (ELU, softmax: the absolute error is then
	// below 1e-7) or feeds a quotient that saturates as |x| grows (TanH, Sigmoid), so results stay
	// inside the 1e-5 relative / 1e-6 absolute tolerance. inf and NaN propagate like expf.
	__device__ __forceinline__ float fast_exp(float x)
	{
		float e;
		asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(x, 1.44269502162933349609375F)));
		return e;
	}

	__device__ __forceinline__ float fast_rcp(float x)
	{
		float r;
		asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
		return r;
	}

	// forward of one activation; `a` = PReLU slope of this element's channel
	template <int KIND>
	__device__ __forceinline__ float act_fwd(float v, float p0, float p1, float a)
	{
		if (KIND == NNF_ACT_RELU)
			return v >= 0.0F ? v : __fmul_rn(v, p0);                 // rectified_linear_layer_tester_plain.cpp:54
		else if (KIND == NNF_ACT_PRELU)
			return __fmul_rn(v, (v >= 0.0F ? 1.0F : a));             // parametric_rectified_linear_layer_tester_plain.cpp:66
		else if (KIND == NNF_ACT_ELU)
			return v >= 0.0F ? v : __fsub_rn(fast_exp(v), 1.0F);     // exponential_linear_layer_tester_plain.cpp:52
		else if (KIND == NNF_ACT_TANH)
		{
			// p0 = scale, p1 = steepness*2 (hyperbolic_tangent_layer_tester_plain.cpp:44-57)
			const float e = fast_exp(__fmul_rn(v, p1));
			const float ep1 = __fadd_rn(e, 1.0F);
			float q = __fmul_rn(__fsub_rn(e, 1.0F), fast_rcp(ep1));
			// the approximate reciprocal flushes to zero above 2^126 where the quotient is exactly 1;
			// e = inf still yields NaN like (inf-1)/(inf+1) does on the CPU
			if (ep1 > 8.0e37F && ep1 < __int_as_float(0x7f800000))
				q = 1.0F;
			return __fmul_rn(q, p0);
		}
		else if (KIND == NNF_ACT_SIGMOID)
			return fast_rcp(__fadd_rn(fast_exp(-v), 1.0F));          // sigmoid_layer_tester_plain.cpp:51
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

	// ---- activation chains (shared by the training batch-norm kernels) ---------------------------
	// Backward through one activation. t_in / t_out are its input and output; the plain backend gates
	// ReLU/PReLU on the input and derives ELU/TanH/Sigmoid from the output.
	template <int KIND>
	__device__ __forceinline__ float act_bwd_one(const act_param& a, float g, float t_in, float t_out, float slope, float& dslope_term)
	{
		if (KIND == NNF_ACT_RELU)
			return act_bwd<NNF_ACT_RELU>(g, t_in, a.p0, 0.0F, 0.0F);
		else if (KIND == NNF_ACT_PRELU)
		{
			// parametric_rectified_linear_layer_updater_plain.cpp:177-180
			dslope_term = __fmul_rn(g, (t_in >= 0.0F ? 0.0F : t_in));
			return act_bwd<NNF_ACT_PRELU>(g, t_in, 0.0F, 0.0F, slope);
		}
		else if (KIND == NNF_ACT_ELU)
			return act_bwd<NNF_ACT_ELU>(g, t_out, 0.0F, 0.0F, 0.0F);
		else if (KIND == NNF_ACT_TANH)
			return act_bwd<NNF_ACT_TANH>(g, t_out, a.p0b, a.p1b, 0.0F);
		else if (KIND == NNF_ACT_SIGMOID)
			return act_bwd<NNF_ACT_SIGMOID>(g, t_out, 0.0F, 0.0F, 0.0F);
		else
			return g;
	}

	__device__ __forceinline__ float act_bwd_one_dyn(const act_param& a, float g, float t_in, float t_out, float slope, float& dslope_term)
	{
		switch (a.kind)
		{
		case NNF_ACT_RELU: return act_bwd_one<NNF_ACT_RELU>(a, g, t_in, t_out, slope, dslope_term);
		case NNF_ACT_PRELU: return act_bwd_one<NNF_ACT_PRELU>(a, g, t_in, t_out, slope, dslope_term);
		case NNF_ACT_ELU: return act_bwd_one<NNF_ACT_ELU>(a, g, t_in, t_out, slope, dslope_term);
		case NNF_ACT_TANH: return act_bwd_one<NNF_ACT_TANH>(a, g, t_in, t_out, slope, dslope_term);
		case NNF_ACT_SIGMOID: return act_bwd_one<NNF_ACT_SIGMOID>(a, g, t_in, t_out, slope, dslope_term);
		default: return g;
		}
	}

	// Recomputes the activation chain from u = x*mult + add, then carries dy back to du.
	// dslope_term receives d(out of PReLU) * (in >= 0 ? 0 : in) for the PReLU in the chain (else 0).
	// A0 >= 0: the chain is known at compile time (A0 then A1, 0 = none); A0 < 0: read from `ch`.
	template <int A0, int A1>
	__device__ __forceinline__ float chain_backward(const act_chain& ch, float u, float dy, float slope, float& dslope_term)
	{
		dslope_term = 0.0F;
		if (A0 >= 0)
		{
			const float t1 = act_fwd<(A0 >= 0 ? A0 : 0)>(u, ch.a[0].p0, ch.a[0].p1, slope);
			float g = dy;
			if (A1 > 0)
			{
				const float t2 = act_fwd<(A1 > 0 ? A1 : 0)>(t1, ch.a[1].p0, ch.a[1].p1, slope);
				g = act_bwd_one<(A1 > 0 ? A1 : 0)>(ch.a[1], g, t1, t2, slope, dslope_term);
			}
			return act_bwd_one<(A0 >= 0 ? A0 : 0)>(ch.a[0], g, u, t1, slope, dslope_term);
		}
		float t[NNF_MAX_ACTS + 1];
		t[0] = u;
		#pragma unroll
		for (int i = 0; i < NNF_MAX_ACTS; ++i)
			t[i + 1] = (i < ch.n) ? act_fwd_dyn(ch.a[i].kind, t[i], ch.a[i].p0, ch.a[i].p1, slope) : t[i];
		float g = dy;
		#pragma unroll
		for (int i = NNF_MAX_ACTS - 1; i >= 0; --i)
			if (i < ch.n)
				g = act_bwd_one_dyn(ch.a[i], g, t[i], t[i + 1], slope, dslope_term);
		return g;
	}

	__device__ __forceinline__ float chain_slope(const act_chain& ch, uint32_t channel)
	{
		float a = 0.0F;
		#pragma unroll
		for (int i = 0; i < NNF_MAX_ACTS; ++i)
			if (i < ch.n && ch.a[i].kind == NNF_ACT_PRELU)
				a = __ldg(ch.a[i].slope + channel);
		return a;
	}


	// forward through the chain; A0 >= 0: compiled-in kinds (A0 then A1, 0 = none), else read from `ch`
	template <int A0, int A1>
	__device__ __forceinline__ float chain_forward(const act_chain& ch, float v, float slope)
	{
		if (A0 >= 0)
		{
			v = act_fwd<(A0 >= 0 ? A0 : 0)>(v, ch.a[0].p0, ch.a[0].p1, slope);
			if (A1 > 0)
				v = act_fwd<(A1 > 0 ? A1 : 0)>(v, ch.a[1].p0, ch.a[1].p1, slope);
			return v;
		}
		else
		{
			#pragma unroll
			for (int i = 0; i < NNF_MAX_ACTS; ++i)
				if (i < ch.n)
					v = act_fwd_dyn(ch.a[i].kind, v, ch.a[i].p0, ch.a[i].p1, slope);
			return v;
		}
	}

	// Chains with a compiled-in fast path: 0 = none, 1 = PReLU then ELU, 2 = ReLU; -1 = generic.
	inline int chain_id(const act_chain& ch)
	{
		if (ch.n == 0)
			return 0;
		if (ch.n == 2 && ch.a[0].kind == NNF_ACT_PRELU && ch.a[1].kind == NNF_ACT_ELU)
			return 1;
		if (ch.n == 1 && ch.a[0].kind == NNF_ACT_RELU)
			return 2;
		return -1;
	}

	// Fills the backward-pass constants of a chain (TanH) from the caller's descriptors.
	inline void chain_fill_backward_constants(act_chain& chain, const nnf_act * acts, int n_acts)
	{
		int j = 0;
		for (int i = 0; i < n_acts && j < chain.n; ++i)
		{
			if (acts[i].kind == NNF_ACT_NONE)
				continue;
			if (acts[i].kind == NNF_ACT_TANH)
			{
				// hyperbolic_tangent_layer_updater_plain.cpp:87-88
				chain.a[j].p0b = 1.0F / acts[i].p0;
				chain.a[j].p1b = acts[i].p1 * acts[i].p0;
			}
			++j;
		}
	}

	// ---- small sums over peer memory (see nnf_peer.cu) ------------------------------------------------
	// Buffer of one rank: float slots[2 parities][kMaxRanks][kmax], then uint32 flags[2][kMaxRanks].
	constexpr int kMaxRanks = 8;
	constexpr uint32_t kPeerSpinLimit = 1u << 22; // x ~200 ns back-off: about a second

	__host__ __device__ inline size_t peer_flags_offset_floats(int kmax) { return size_t(2) * kMaxRanks * kmax; }

	struct peer_src           // where a kernel finds the messages of all ranks (its OWN buffer)
	{
		const float * mine;   // null: no peer exchange, read the plain sums buffer instead
		int world;
		int kmax;
		uint32_t seq;
		int * error;
	};

	struct peer_dst           // where a kernel publishes this rank's message (EVERY rank's buffer)
	{
		float * base[kMaxRanks];
		int rank;
		int world;            // 0: do not publish
		int kmax;
		uint32_t seq;
	};

	// Called by all threads of a CTA: the first `world` threads wait (bounded) for the flags of this
	// exchange in the rank's own buffer; on expiry the error word is raised and the kernel carries on.
	__device__ __forceinline__ void peer_wait(const peer_src& s)
	{
		if ((int)threadIdx.x < s.world)
		{
			const uint32_t * flag = reinterpret_cast<const uint32_t *>(s.mine + peer_flags_offset_floats(s.kmax)) + (s.seq & 1u) * kMaxRanks + threadIdx.x;
			uint32_t seen = 0;
			bool ok = false;
			for (uint32_t i = 0; i < kPeerSpinLimit; ++i)
			{
				asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
				if (seen == s.seq)
				{
					ok = true;
					break;
				}
				__nanosleep(200);
			}
			if (!ok && s.error)
				*s.error = 2;
		}
		__syncthreads();
	}

	// sum over ranks, in rank order, of element `index` of the published messages
	__device__ __forceinline__ float peer_sum(const peer_src& s, uint32_t index)
	{
		float t = 0.0F;
		for (int r = 0; r < s.world; ++r)
			t += __ldcv(s.mine + (size_t(s.seq & 1u) * kMaxRanks + r) * s.kmax + index);
		return t;
	}

	// Called by all threads of the (single) publishing CTA after their peer stores.
	__device__ __forceinline__ void peer_raise_flags(const peer_dst& d)
	{
		__threadfence_system();
		__syncthreads();
		if ((int)threadIdx.x < d.world)
		{
			uint32_t * flag = reinterpret_cast<uint32_t *>(d.base[threadIdx.x] + peer_flags_offset_floats(d.kmax)) + (d.seq & 1u) * kMaxRanks + d.rank;
			asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flag), "r"(d.seq) : "memory");
		}
	}

	__device__ __forceinline__ void peer_store(const peer_dst& d, uint32_t index, float v)
	{
		for (int r = 0; r < d.world; ++r)
			d.base[r][(size_t(d.seq & 1u) * kMaxRanks + d.rank) * d.kmax + index] = v;
	}

	int make_peer_dst(peer_dst& d, void * const * peer_bufs, int rank, int world, int k, int kmax, uint32_t seq, const char * who);
	int * device_error_word();

	// workspace of the single-launch training batch norm (nnf_bn_chain.cu)
	size_t chain_workspace_bytes(int64_t n, int64_t c, int64_t hw);

	// ---- memory access helpers -----------------------------------------------------------------
	// Streaming (evict-first) 128-bit accesses: every tensor on this path is touched once per kernel.
	__device__ __forceinline__ float4 ld_stream(const float4 * p) { return __ldcs(p); }
	__device__ __forceinline__ void st_stream(float4 * p, float4 v) { __stcs(p, v); }
	__device__ __forceinline__ float ld_stream(const float * p) { return __ldcs(p); }
	__device__ __forceinline__ void st_stream(float * p, float v) { __stcs(p, v); }

	inline bool aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

	inline int64_t div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }
}
