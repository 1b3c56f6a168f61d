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

	// A schema in text form, one layer per line: "name type inputs [needed] [key=value ...]" with inputs a
	// comma-separated list of layer names or "-" for none. Keys: alpha (Add, AverageSubsampling), slope (ReLU),
	// scale and steepness (TanH; scale also NegativeLogLikelihood), eps (BatchNorm), topn (Accuracy),
	// win / stride / roundup (subsampling, e.g. win=3x3 stride=2x2 roundup=0x0), min, fm (feature-map
	// subsampling size), tiling. Stands in for the protobuf schema of the reference in tests and examples.
	std::vector<schema_node> parse_schema(const std::string& spec);
}
