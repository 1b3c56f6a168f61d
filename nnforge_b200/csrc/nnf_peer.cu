// Small all-reduce (sum) over peer memory for the 2*C-float statistics messages of batch-sharded
// training batch norm. Each rank owns one buffer that every peer can address (symmetric memory: the
// caller maps it, e.g. torch.distributed._symmetric_memory, and passes the per-rank base pointers).
//
//   publish: this rank stores its K floats into slot [parity][rank] of EVERY rank's buffer (plain
//            coalesced peer stores over NVLink), fences, then raises flag [parity][rank] = seq on every rank;
//   gather : waits - bounded - until all `world` flags of its OWN buffer show seq, then sums the slots in
//            rank order (identical result on every rank).
// Both are single-CTA kernels on the caller's stream, so the exchange costs two ~2 us launches plus one
// NVLink store latency instead of an NCCL all-reduce launch (~20 us for 2 KB on this machine). Slots are
// double-buffered by the parity of seq: a rank can only publish exchange k+2 after it gathered k+1, which
// needed every peer's publish k+1, which follows that peer's gather k in stream order.
//
// The wait is on the rank's own memory, bounded (about a second), and on expiry raises an error word and
// lets the kernel finish; nothing spins forever and no peer memory is ever read.
#include "nnf_common.cuh"

#include <mutex>

namespace nnf
{
	namespace
	{
		constexpr int kPeerThreads = 1024;

		__global__ void __launch_bounds__(kPeerThreads) peer_publish_kernel(const float * local, peer_dst dst, int k)
		{
			for (int i = threadIdx.x; i < k; i += kPeerThreads)
				peer_store(dst, i, local[i]);
			peer_raise_flags(dst);
		}

		__global__ void __launch_bounds__(kPeerThreads) peer_gather_sum_kernel(float * out, peer_src src, int k)
		{
			peer_wait(src);
			for (int i = threadIdx.x; i < k; i += kPeerThreads)
				out[i] = peer_sum(src, i);
		}
	}

	int make_peer_dst(peer_dst& d, void * const * peer_bufs, int rank, int world, int k, int kmax, uint32_t seq, const char * who)
	{
		if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: rank %d of %d (at most %d ranks)", who, rank, world, kMaxRanks);
		if (k < 1 || kmax < k)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: %d floats do not fit slots of %d", who, k, kmax);
		if (!peer_bufs || seq == 0)
			return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: null pointer table or seq 0 (sequence numbers start at 1; the buffers start zeroed)", who);
		for (int r = 0; r < kMaxRanks; ++r)
			d.base[r] = nullptr;
		for (int r = 0; r < world; ++r)
		{
			if (!peer_bufs[r])
				return set_error(NNF_ERR_INVALID_ARGUMENT, "%s: buffer of rank %d is null", who, r);
			d.base[r] = static_cast<float *>(peer_bufs[r]);
		}
		d.rank = rank; d.world = world; d.kmax = kmax; d.seq = seq;
		return NNF_OK;
	}
}

using namespace nnf;

extern "C" size_t nnf_peer_exchange_bytes(int kmax)
{
	if (kmax < 1)
		return 0;
	return (peer_flags_offset_floats(kmax) + size_t(2) * kMaxRanks) * sizeof(float);
}

extern "C" int nnf_peer_publish(nnf_stream_t stream, const float * local, void * const * peer_bufs, int rank, int world, int k, int kmax, uint32_t seq)
{
	peer_dst d;
	int st = make_peer_dst(d, peer_bufs, rank, world, k, kmax, seq, "nnf_peer_publish");
	if (st != NNF_OK)
		return st;
	if (!local)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_peer_publish: null message");
	peer_publish_kernel<<<1, kPeerThreads, 0, (cudaStream_t)stream>>>(local, d, k);
	return check_launch("peer_publish_kernel");
}

extern "C" int nnf_peer_gather_sum(nnf_stream_t stream, float * out, const void * my_buf, int world, int k, int kmax, uint32_t seq)
{
	if (world < 1 || world > kMaxRanks || k < 1 || kmax < k || !out || !my_buf || seq == 0)
		return set_error(NNF_ERR_INVALID_ARGUMENT, "nnf_peer_gather_sum: bad arguments (world %d, k %d, kmax %d)", world, k, kmax);
	peer_src src;
	src.mine = static_cast<const float *>(my_buf); src.world = world; src.kmax = kmax; src.seq = seq; src.error = device_error_word();
	peer_gather_sum_kernel<<<1, kPeerThreads, 0, (cudaStream_t)stream>>>(out, src, k);
	return check_launch("peer_gather_sum_kernel");
}

extern "C" int nnf_peer_exchange_sum(nnf_stream_t stream, float * out, const float * local, void * const * peer_bufs, int rank, int world, int k, int kmax, uint32_t seq)
{
	int st = nnf_peer_publish(stream, local, peer_bufs, rank, world, k, kmax, seq);
	if (st != NNF_OK)
		return st;
	return nnf_peer_gather_sum(stream, out, peer_bufs[rank], world, k, kmax, seq);
}
