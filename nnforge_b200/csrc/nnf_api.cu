// Status text and version entry points of the C ABI.
#include "nnf_common.cuh"

#include <stdarg.h>

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

extern "C" const char * nnf_last_error_string(void)
{
	return nnf::g_error;
}

extern "C" int nnf_version(void)
{
	return 100;
}
