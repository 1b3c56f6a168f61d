// Status text and version entry points of the C ABI.
#include "nnf_common.cuh"

#include <stdarg.h>
#include <string.h>

#include <mutex>

namespace nnf
{
	namespace
	{
		thread_local char g_error[512] = "";
	}

	int set_error(int status, const char * fmt, ...)
	{
		va_list ap;
		va_start(ap, fmt);
		vsnprintf(g_error, sizeof(g_error), fmt, ap);
		va_end(ap);
		return status;
	}

	int check_launch(const char * what)
	{
		cudaError_t e = cudaGetLastError();
		if (e != cudaSuccess)
			return set_error(NNF_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
		return NNF_OK;
	}
}

namespace nnf
{
	const running_configuration& running_config()
	{
		static std::mutex mu;
		static running_configuration cfg[64];
		static bool filled[64] = {};
		int dev = 0;
		if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
			dev = 0;
		std::lock_guard<std::mutex> lock(mu);
		if (!filled[dev])
		{
			running_configuration& r = cfg[dev];
			r.device_id = dev;
			auto attr = [&](cudaDeviceAttr a, int fallback) { int v = 0; return cudaDeviceGetAttribute(&v, a, dev) == cudaSuccess && v > 0 ? v : fallback; };
			// the fallbacks are B200's figures: they are used only where the query itself fails (no device at build checks)
			r.compute_capability_major = attr(cudaDevAttrComputeCapabilityMajor, 10);
			r.compute_capability_minor = attr(cudaDevAttrComputeCapabilityMinor, 0);
			r.multiprocessor_count = attr(cudaDevAttrMultiProcessorCount, 148);
			r.max_threads_per_multiprocessor = attr(cudaDevAttrMaxThreadsPerMultiProcessor, 2048);
			r.max_shared_memory_per_block_optin = attr(cudaDevAttrMaxSharedMemoryPerBlockOptin, 227 * 1024);
			r.max_shared_memory_per_multiprocessor = attr(cudaDevAttrMaxSharedMemoryPerMultiprocessor, 228 * 1024);
			r.l2_cache_size = attr(cudaDevAttrL2CacheSize, 126 * 1024 * 1024);
			r.max_registers_per_multiprocessor = attr(cudaDevAttrMaxRegistersPerMultiprocessor, 65536);
			cudaGetLastError();
			filled[dev] = true;
		}
		return cfg[dev];
	}

	tuning& tune()
	{
		static tuning t = {0, 0, 0, 0, 0, 0, 0, 0, -1, 0, 0, 0, 0, 0};
		return t;
	}
}

extern "C" int nnf_get_running_configuration(nnf_running_configuration * out)
{
	if (!out)
		return nnf::set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_get_running_configuration: null pointer");
	const nnf::running_configuration& r = nnf::running_config();
	out->device_id = r.device_id;
	out->compute_capability_major = r.compute_capability_major;
	out->compute_capability_minor = r.compute_capability_minor;
	out->multiprocessor_count = r.multiprocessor_count;
	out->max_threads_per_multiprocessor = r.max_threads_per_multiprocessor;
	out->max_shared_memory_per_block_optin = r.max_shared_memory_per_block_optin;
	out->max_shared_memory_per_multiprocessor = r.max_shared_memory_per_multiprocessor;
	out->l2_cache_size = r.l2_cache_size;
	out->max_registers_per_multiprocessor = r.max_registers_per_multiprocessor;
	return NNF_OK;
}

extern "C" int nnf_set_tuning(const char * name, long long value)
{
	if (!name)
		return nnf::set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_set_tuning: null name");
	nnf::tuning& t = nnf::tune();
	struct entry { const char * name; int * field; };
	const entry table[] = {
		{"elementwise_waves", &t.elementwise_waves}, {"elementwise_group_waves", &t.elementwise_group_waves},
		{"pool_waves", &t.pool_waves}, {"pool_group_floats", &t.pool_group_floats},
		{"channel_waves", &t.channel_waves}, {"group_waves", &t.group_waves},
		{"chain_s_kb", &t.chain_s_kb}, {"chain_a_kb", &t.chain_a_kb}, {"chain_dist", &t.chain_dist},
		{"chain_chunk_mb", &t.chain_chunk_mb}, {"chain_lag", &t.chain_lag},
		{"no_grouped", &t.no_grouped}, {"apply_flat", &t.apply_flat},
	};
	if (strcmp(name, "peer_wait_ns") == 0)
	{
		t.peer_wait_ns = value;
		return NNF_OK;
	}
	if (strcmp(name, "reset") == 0)
	{
		t = nnf::tuning{0, 0, 0, 0, 0, 0, 0, 0, -1, 0, 0, 0, 0, 0};
		return NNF_OK;
	}
	for (const entry& e : table)
		if (strcmp(name, e.name) == 0)
		{
			*e.field = (int)value;
			return NNF_OK;
		}
	return nnf::set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_set_tuning: unknown knob '%s'", name);
}

extern "C" const char * nnf_last_error_string(void)
{
	return nnf::g_error;
}

extern "C" int nnf_version(void)
{
	return 100;
}
