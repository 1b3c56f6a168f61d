// Helpers shared by the translation units that implement the host-side layer objects: status check of a
// C-ABI call, pointer access to scheduler buffers, and the translation of layer parameters into the
// C ABI's activation and pooling descriptors. Not part of the interface.
#pragma once

#include "nnf_layers.h"

#include "../../../include/nnf_b200.h"

#include <cstring>

namespace nnf_b200
{
namespace detail
{
	inline void check(int status)
	{
		if (status != NNF_OK)
			throw neural_network_exception(std::string("nnf_b200: ") + nnf_last_error_string());
	}

	inline const float * f(const device_buffer::const_ptr& b) { return b ? static_cast<const float *>(*b) : nullptr; }
	inline float * f(const device_buffer::ptr& b) { return b ? static_cast<float *>(*b) : nullptr; }

	inline nnf_act make_act(const layer& l, const float * slope)
	{
		nnf_act a;
		a.kind = NNF_ACT_NONE; a.p0 = 0.0F; a.p1 = 0.0F; a.slope = slope;
		if (l.type_name == "ReLU") { a.kind = NNF_ACT_RELU; a.p0 = l.negative_slope; }
		else if (l.type_name == "PReLU") a.kind = NNF_ACT_PRELU;
		else if (l.type_name == "ELU") a.kind = NNF_ACT_ELU;
		else if (l.type_name == "TanH") { a.kind = NNF_ACT_TANH; a.p0 = l.scale; a.p1 = l.steepness; }
		else if (l.type_name == "Sigmoid") a.kind = NNF_ACT_SIGMOID;
		return a;
	}

	// ReLU/PReLU read their input in backward, the other three their output (the plain backend's dependencies)
	inline bool backward_uses_input(const layer& l) { return l.type_name == "ReLU" || l.type_name == "PReLU"; }

	inline nnf_pool make_pool(const layer& l, const layer_configuration_specific& in)
	{
		if (l.tiling)
			throw neural_network_exception("max subsampling with tiling is not supported"); // the reference updater refuses it too
		if (l.feature_map_subsampling_size != 1 || l.entry_subsampling_size != 1)
			throw neural_network_exception("max subsampling over feature maps or entries is not supported");
		if (l.subsampling_sizes.empty() || l.subsampling_sizes.size() > 2 || l.subsampling_sizes.size() != in.dimension_sizes.size())
			throw neural_network_exception("max subsampling supports 1 or 2 spatial dimensions matching the input");
		nnf_pool p;
		std::memset(&p, 0, sizeof(p));
		p.win_w = (int)l.subsampling_sizes[0];
		p.stride_w = l.strides.empty() ? p.win_w : (int)l.strides[0];
		p.round_up_w = (!l.round_ups.empty() && l.round_ups[0]) ? 1 : 0;
		p.win_h = p.stride_h = 1;
		if (l.subsampling_sizes.size() == 2)
		{
			p.win_h = (int)l.subsampling_sizes[1];
			p.stride_h = l.strides.size() > 1 ? (int)l.strides[1] : p.win_h;
			p.round_up_h = (l.round_ups.size() > 1 && l.round_ups[1]) ? 1 : 0;
		}
		p.is_min = l.is_min ? 1 : 0;
		return p;
	}

	inline unsigned int dim(const layer_configuration_specific& c, size_t i) { return i < c.dimension_sizes.size() ? c.dimension_sizes[i] : 1; }

	inline bool is_activation(const std::string& t) { return t == "ReLU" || t == "PReLU" || t == "ELU" || t == "TanH" || t == "Sigmoid"; }

	inline void * raw(const device_buffer::ptr& b) { return b ? static_cast<void *>(*b) : nullptr; }

	// what the flat driver interface (nnfh_*) hands out as an opaque pointer: one layer object of either kind
	struct flat_handle
	{
		std::shared_ptr<layer> schema;
		layer_tester_b200::ptr tester;
		layer_updater_b200::ptr updater;
		std::vector<device_buffer::ptr> uploaded;               // what get_data / set_get_data_custom returned, kept alive
		std::vector<device_buffer::const_ptr> uploaded_const;
	};

	// the training batch-norm object that also runs the activation layers given (the head of a fused group)
	layer_updater_b200::ptr make_batch_norm_updater(const std::vector<layer>& followers);
}
}
