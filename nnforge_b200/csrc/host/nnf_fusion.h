// Peephole over a layer schema: which runs of nnForge layers one fused entry point of the C ABI can execute, and
// which intermediate buffers then never have to exist. This is the decision that the reference's schedulers would
// take in forward_propagation_cuda::layer_config_map_modified / backward_propagation_cuda (they create one
// tester / updater object per layer and one buffer per layer output, nnforge/cuda/forward_propagation_cuda.cpp:726-890);
// it is kept free of any scheduler type so that it can be tested on its own and called from there.
//
// Patterns (a run is only fused through a layer output that has exactly one reader and is not needed elsewhere):
//   inference   [BatchNorm] -> [Add with one other input] -> up to two activations          nnf_bn_infer_act
//               ... -> one ReLU -> MaxSubsampling (2-D windows)                              nnf_bn_add_relu_maxpool_fwd
//               ... -> one ReLU -> AverageSubsampling (2-D windows)                          nnf_bn_add_relu_avgpool_fwd
//               (the pooled forms write the ReLU output z themselves, so z may have other readers)
//   training    BatchNorm -> up to two activations (at most one PReLU)                       nnf_bn_train_fwd / nnf_bn_train_bwd
//   both        Softmax -> NegativeLogLikelihood (input 0)                                   nnf_softmax_nll_fwd / _bwd
//               (the probabilities are written, so Softmax may have other readers, e.g. Accuracy)
#pragma once

#include "nnf_layers.h"

#include <string>
#include <vector>

namespace nnf_b200
{
	struct schema_node
	{
		std::string name;                  // layer instance name
		layer params;                      // type name and parameters
		std::vector<std::string> inputs;   // instance names of the layers whose outputs it reads (none: data layer)
		bool output_needed = false;        // its output is read outside this list (network output, kept for another pass)
	};

	enum fused_kind
	{
		fused_single_layer = 0,
		fused_bn_act,
		fused_bn_add_relu_maxpool,
		fused_bn_add_relu_avgpool,
		fused_bn_train_act,
		fused_softmax_nll
	};

	struct fused_group
	{
		fused_kind kind = fused_single_layer;
		std::vector<int> members;          // node indices in execution order; the last one's output is the group's output
		int bn = -1, add = -1, pool = -1, softmax = -1, loss = -1;
		std::vector<int> acts;
		std::string residual_input;        // the Add's other input, when the group contains an Add
		std::string entry_point;           // C-ABI call that runs the group's forward pass
		std::vector<int> elided;           // members whose output buffer is never materialised
	};

	// nodes must be in execution (topological) order. Every node ends up in exactly one group.
	std::vector<fused_group> plan_fusion(const std::vector<schema_node>& nodes, bool training);

	// The objects that run the plan are made by layer_factory_b200::create_testers / create_updaters (nnf_layers.h).

	// Which layer outputs of an inference schedule share storage: the part of network_action_schema::get_buffer_set
	// (nnforge/network_action_schema.h:106-109, driven from forward_propagation_cuda::setup_layer_buffer_sizes,
	// nnforge/cuda/forward_propagation_cuda.cpp:771-832) that a scheduler needs once groups are fused. Actions run in the order of
	// the node list, a fused group at the position of its first member. A materialised output lives from the action that writes it
	// to the last action that reads it (to the end when output_needed); outputs in fused_group::elided get no buffer; an object whose
	// get_input_index_layer_can_write() names an input writes its (first) output over that input's buffer when nobody reads the
	// input afterwards; otherwise an output takes the smallest free buffer that is large enough, or a new one.
	struct buffer_plan
	{
		std::vector<int> buffer_of_node;              // per node: index of its output's buffer, -1 for an elided output
		std::vector<size_t> buffer_bytes_per_entry;   // per buffer
		std::vector<int> written_in_place;            // per node: the input index whose buffer the output took over, or -1
		size_t total_bytes_per_entry = 0;
	};
	// can_write[i]: what the object that runs node i answers (the head's answer for the first member of a group; ignored for the other
	// members). output_bytes_per_entry[i]: size of node i's output.
	buffer_plan plan_forward_buffers(const std::vector<schema_node>& nodes, const std::vector<fused_group>& groups,
		const std::vector<int>& can_write, const std::vector<size_t>& output_bytes_per_entry);

	// A schema in text form, one layer per line: "name type inputs [needed] [key=value ...]" with inputs a
	// comma-separated list of layer names or "-" for none. Keys: alpha (Add, AverageSubsampling), slope (ReLU),
	// scale and steepness (TanH; scale also NegativeLogLikelihood), eps (BatchNorm), topn (Accuracy),
	// win / stride / roundup (subsampling, e.g. win=3x3 stride=2x2 roundup=0x0), min, fm (feature-map
	// subsampling size), tiling. Stands in for the protobuf schema of the reference in tests and examples.
	std::vector<schema_node> parse_schema(const std::string& spec);
}
