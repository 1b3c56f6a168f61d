// The objects that run a planned fused group (nnf_fusion.h) behind the per-layer interface of nnf_layers.h:
// one head per group, which calls the group's fused entry point of the C ABI, and no-op followers for the other
// members - plus layer_factory_b200::create_testers / create_updaters, which build them from a fused_group, and
// a flat driver (nnfh_net_*) that builds the objects of a whole textual schema for the tests and the benchmark.
//
// What a scheduler does differently for a fused group than for stock layers (nnforge/cuda/forward_propagation_cuda.cpp:726-890
// creates one tester and one output buffer per layer and enqueues them in action order):
//   - the head is enqueued where the group's first member would run, with the inputs, weight chunks and output
//     buffers that fused_io names; the followers are enqueued as usual and do nothing;
//   - outputs listed in fused_group::elided need no buffer (a per-layer buffer plan that keeps them puts them on the
//     head's buffer, because every follower of a chain answers get_input_index_layer_can_write() == 0);
//   - in training, the weight gradients of a fused PReLU are written by the head's backward action, so the follower's
//     update_weights action has to wait for that action, not for the follower's own (empty) backward_weights action.
#include "nnf_fusion.h"
#include "nnf_layers_detail.h"

#include <sstream>

namespace nnf_b200
{
	using namespace detail;

	namespace
	{
		// ---- followers ----------------------------------------------------------------------------
		class fused_follower_tester_b200 : public layer_tester_b200
		{
		public:
			explicit fused_follower_tester_b200(bool in_place) : in_place(in_place) {}
			void enqueue_forward_propagation(cudaStream_t, device_buffer::ptr, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int) override
			{
				// the head of the group has written this layer's output already, or nobody reads it
			}
			int get_input_index_layer_can_write() const override { return in_place ? 0 : -1; }
		private:
			bool in_place;
		};

		class fused_follower_updater_b200 : public layer_updater_b200
		{
		public:
			explicit fused_follower_updater_b200(bool in_place) : in_place(in_place) {}
			void enqueue_forward_propagation(cudaStream_t, device_buffer::ptr, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int) override
			{
			}
			// The error of the group's output reaches the head unchanged: in place, this layer's input errors ARE its output errors.
			void enqueue_backward_data_propagation(cudaStream_t, unsigned int, device_buffer::ptr input_errors_buffer, device_buffer::const_ptr output_errors_buffer,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr, const std::vector<device_buffer::const_ptr>&, device_buffer::ptr,
				device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr, bool, unsigned int) override
			{
				if (in_place && input_errors_buffer && output_errors_buffer
					&& static_cast<const void *>(*output_errors_buffer) != static_cast<void *>(*input_errors_buffer))
					throw neural_network_exception("follower of a fused group (" + layer_schema->type_name
						+ "): its input errors must share the buffer of its output errors, as get_input_index_layer_can_write() asks");
			}
			// a fused PReLU's slope gradient is accumulated by the head's backward action
			void enqueue_backward_weights_propagation(cudaStream_t, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				unsigned int) override
			{
			}
			int get_input_index_layer_can_write(const layer_action& action) const override
			{
				return (in_place && (action.get_action_type() == layer_action::forward || action.get_action_type() == layer_action::backward_data)) ? 0 : -1;
			}
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return false; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return false; }
			bool is_backward_weights_dependent_on_input_buffer(unsigned int) const override { return false; }
		private:
			bool in_place;
		};

		// ---- heads: inference ---------------------------------------------------------------------
		// What the inference heads share: [BatchNorm] -> [Add] -> activations, read from the group description.
		struct chain_description
		{
			bool has_bn = false, has_add = false;
			float add_alpha = 1.0F;
			std::vector<layer> acts;

			size_t chunk_count() const
			{
				size_t n = has_bn ? 4 : 0;
				for (const layer& l : acts)
					n += l.type_name == "PReLU";
				return n;
			}
			size_t input_count() const { return has_add ? 2 : 1; }
			void check_lists(const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>& input_buffers, const char * who) const
			{
				if (data.size() != chunk_count())
					throw neural_network_exception(std::string(who) + ": " + std::to_string(chunk_count()) + " weight chunks expected (batch norm's four, then one per PReLU), "
						+ std::to_string(data.size()) + " given");
				if (input_buffers.size() != input_count())
					throw neural_network_exception(std::string(who) + ": " + std::to_string(input_count()) + " input buffers expected, " + std::to_string(input_buffers.size()) + " given");
			}
			std::vector<nnf_act> make_acts(const std::vector<device_buffer::const_ptr>& data) const
			{
				std::vector<nnf_act> res;
				size_t chunk = has_bn ? 4 : 0;
				for (const layer& l : acts)
					res.push_back(make_act(l, l.type_name == "PReLU" ? f(data[chunk++]) : nullptr));
				return res;
			}
		};

		// nnf_bn_infer_act: one pass for the whole chain
		class fused_bn_act_tester_b200 : public layer_tester_b200
		{
		public:
			explicit fused_bn_act_tester_b200(const chain_description& chain) : chain(chain) {}
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				chain.check_lists(data, input_buffers, "fused BatchNorm/Add/activation tester");
				const std::vector<nnf_act> acts = chain.make_acts(data);
				check(nnf_bn_infer_act(stream_id, f(output_buffer), f(input_buffers[0]),
					chain.has_bn ? f(data[0]) : nullptr, chain.has_bn ? f(data[1]) : nullptr, chain.has_bn ? f(data[2]) : nullptr, chain.has_bn ? f(data[3]) : nullptr,
					chain.has_add ? f(input_buffers[1]) : nullptr, chain.add_alpha, acts.empty() ? nullptr : acts.data(), (int)acts.size(),
					entry_count, output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			int get_input_index_layer_can_write() const override { return 0; }
		private:
			chain_description chain;
		};

		// nnf_bn_add_relu_maxpool_fwd / nnf_bn_add_relu_avgpool_fwd: writes the ReLU output z and the pooled tensor
		class fused_pooled_tester_b200 : public layer_tester_b200
		{
		public:
			fused_pooled_tester_b200(const chain_description& chain, const layer& pool_layer, bool average) : chain(chain), pool_layer(pool_layer), average(average) {}
			void enqueue_forward_propagation(cudaStream_t, device_buffer::ptr, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int) override
			{
				throw neural_network_exception("the head of a fused pooling group writes two outputs: call enqueue_forward_propagation with the list {ReLU output, pooled output}");
			}
			void enqueue_forward_propagation(cudaStream_t stream_id, const std::vector<device_buffer::ptr>& output_buffers, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (output_buffers.size() != 2 || !output_buffers[0] || !output_buffers[1])
					throw neural_network_exception("the head of a fused pooling group needs two output buffers: the ReLU output and the pooled output");
				chain.check_lists(data, input_buffers, "fused pooling tester");
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				const float * gamma = chain.has_bn ? f(data[0]) : nullptr, * beta = chain.has_bn ? f(data[1]) : nullptr;
				const float * mean = chain.has_bn ? f(data[2]) : nullptr, * invsigma = chain.has_bn ? f(data[3]) : nullptr;
				const float * residual = chain.has_add ? f(input_buffers[1]) : nullptr;
				const float slope = chain.acts.at(0).negative_slope;
				if (average)
					check(nnf_bn_add_relu_avgpool_fwd(stream_id, f(output_buffers[0]), f(output_buffers[1]), f(input_buffers[0]), residual, gamma, beta, mean, invsigma, slope,
						entry_count, in.feature_map_count, dim(in, 1), dim(in, 0), (int)pool_layer.subsampling_sizes.at(0), (int)pool_layer.subsampling_sizes.at(1), pool_layer.alpha));
				else
					check(nnf_bn_add_relu_maxpool_fwd(stream_id, f(output_buffers[0]), f(output_buffers[1]), nullptr, f(input_buffers[0]), residual, gamma, beta, mean, invsigma, slope,
						entry_count, in.feature_map_count, dim(in, 1), dim(in, 0), &pool));
			}
			unsigned int get_output_count() const override { return 2; }
			int get_input_index_layer_can_write() const override { return 0; } // z may take the place of x
		protected:
			void tester_configured() override
			{
				if (!average)
					pool = make_pool(pool_layer, input_configuration_specific_list[0]);
			}
		private:
			chain_description chain;
			layer pool_layer;
			bool average;
			nnf_pool pool;
		};

		// nnf_softmax_nll_fwd: probabilities and the loss in one pass. inputs = logits, targets[, scale mask]
		class fused_softmax_nll_tester_b200 : public layer_tester_b200
		{
		public:
			explicit fused_softmax_nll_tester_b200(float scale) : scale(scale) {}
			void enqueue_forward_propagation(cudaStream_t, device_buffer::ptr, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int) override
			{
				throw neural_network_exception("the head of a fused softmax + loss group writes two outputs: call enqueue_forward_propagation with the list {probabilities, loss}");
			}
			void enqueue_forward_propagation(cudaStream_t stream_id, const std::vector<device_buffer::ptr>& output_buffers, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (output_buffers.size() != 2 || input_buffers.size() < 2)
					throw neural_network_exception("fused softmax + loss: outputs {probabilities, loss} and inputs {logits, targets[, mask]} expected");
				check(nnf_softmax_nll_fwd(stream_id, f(output_buffers[0]), f(output_buffers[1]), f(input_buffers[0]), f(input_buffers[1]),
					input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr, scale, entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			unsigned int get_output_count() const override { return 2; }
		private:
			float scale;
		};

		// ---- heads: training ----------------------------------------------------------------------
		// (BatchNorm -> activations is batch_norm_layer_updater_b200 itself, given the followers: make_batch_norm_updater)
		class fused_softmax_nll_updater_b200 : public layer_updater_b200
		{
		public:
			explicit fused_softmax_nll_updater_b200(float scale) : scale(scale) {}
			void enqueue_forward_propagation(cudaStream_t, device_buffer::ptr, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int) override
			{
				throw neural_network_exception("the head of a fused softmax + loss group writes two outputs: call enqueue_forward_propagation with the list {probabilities, loss}");
			}
			void enqueue_forward_propagation(cudaStream_t stream_id, const std::vector<device_buffer::ptr>& output_buffers, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (output_buffers.size() != 2 || input_buffers.size() < 2)
					throw neural_network_exception("fused softmax + loss: outputs {probabilities, loss} and inputs {logits, targets[, mask]} expected");
				check(nnf_softmax_nll_fwd(stream_id, f(output_buffers[0]), f(output_buffers[1]), f(input_buffers[0]), f(input_buffers[1]),
					input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr, scale, entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			// the loss has no output errors: the gradient of the logits comes from the probabilities and the targets
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int input_index, device_buffer::ptr input_errors_buffer, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_neurons_buffers, device_buffer::const_ptr output_neurons_buffer,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				if (input_index != 0)
					throw neural_network_exception("fused softmax + loss cannot do backward propagation for targets or the scale mask");
				if (input_neurons_buffers.size() < 2 || !output_neurons_buffer)
					throw neural_network_exception("fused softmax + loss backward needs the probabilities (output neurons) and the targets (input 1)");
				check(nnf_softmax_nll_bwd(stream_id, f(input_errors_buffer), f(output_neurons_buffer), f(input_neurons_buffers[1]),
					input_neurons_buffers.size() > 2 ? f(input_neurons_buffers[2]) : nullptr, scale, entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map, add_update_to_destination ? 1 : 0));
			}
			unsigned int get_output_count() const override { return 2; }
			// the logits are not read again; targets and mask are
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int data_input_index) const override { return data_input_index != 0; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return true; }
		private:
			float scale;
		};

		// ---- building the objects of a group --------------------------------------------------------
		const layer_configuration_specific& shape_of(const std::map<std::string, layer_configuration_specific>& shapes, const std::string& name)
		{
			auto it = shapes.find(name);
			if (it == shapes.end())
				throw neural_network_exception("No output configuration given for layer " + name);
			return it->second;
		}

		unsigned int input_index_of(const schema_node& n, const std::string& input_name)
		{
			for (size_t k = 0; k < n.inputs.size(); ++k)
				if (n.inputs[k] == input_name)
					return (unsigned int)k;
			throw neural_network_exception("Layer " + n.name + " does not read " + input_name);
		}

		// inputs, weight chunks and outputs of the group's head; also the chain description for the inference kinds
		fused_io describe_group(const fused_group& g, const std::vector<schema_node>& nodes, chain_description& chain)
		{
			fused_io io;
			const int head = g.members.at(0);
			if (g.kind == fused_single_layer)
			{
				for (size_t k = 0; k < nodes[head].inputs.size(); ++k)
					io.input_sources.push_back(std::make_pair(head, (unsigned int)k));
				io.data_sources.push_back(head);
				io.output_sources.push_back(head);
				return io;
			}
			if (g.kind == fused_softmax_nll)
			{
				io.input_sources.push_back(std::make_pair(g.softmax, 0U));
				for (size_t k = 1; k < nodes[g.loss].inputs.size(); ++k)
					io.input_sources.push_back(std::make_pair(g.loss, (unsigned int)k));
				io.output_sources = {g.softmax, g.loss};
				return io;
			}
			chain.has_bn = g.bn >= 0;
			chain.has_add = g.add >= 0;
			io.input_sources.push_back(std::make_pair(head, head == g.add ? 1U - input_index_of(nodes[head], g.residual_input) : 0U));
			if (g.add >= 0)
			{
				chain.add_alpha = nodes[g.add].params.alpha;
				io.input_sources.push_back(std::make_pair(g.add, input_index_of(nodes[g.add], g.residual_input)));
			}
			if (g.bn >= 0)
				io.data_sources.push_back(g.bn);
			for (int a : g.acts)
			{
				chain.acts.push_back(nodes[a].params);
				if (nodes[a].params.type_name == "PReLU")
					io.data_sources.push_back(a);
			}
			if (g.kind == fused_bn_add_relu_maxpool || g.kind == fused_bn_add_relu_avgpool)
				io.output_sources = {g.acts.at(0), g.pool};
			else
				io.output_sources = {g.members.back()};
			return io;
		}

		std::vector<layer_configuration_specific> input_shapes(const fused_io& io, const std::vector<schema_node>& nodes,
			const std::map<std::string, layer_configuration_specific>& shapes)
		{
			std::vector<layer_configuration_specific> res;
			for (const auto& src : io.input_sources)
				res.push_back(shape_of(shapes, nodes[src.first].inputs.at(src.second)));
			return res;
		}

		std::vector<layer_configuration_specific> own_input_shapes(const schema_node& n, const std::map<std::string, layer_configuration_specific>& shapes)
		{
			std::vector<layer_configuration_specific> res;
			for (const std::string& in : n.inputs)
				res.push_back(shape_of(shapes, in));
			return res;
		}

		// a follower stays on the buffer of the member before it when it is a link of the chain (same shape, one input);
		// the pooling layer and the loss have outputs of their own, which the head writes
		bool follower_in_place(const fused_group& g, int member)
		{
			return member != g.pool && member != g.loss;
		}
	}

	fused_testers layer_factory_b200::create_testers(const fused_group& g, const std::vector<schema_node>& nodes,
		const std::map<std::string, layer_configuration_specific>& shapes, running_configuration_b200::const_ptr cuda_config) const
	{
		if (g.members.empty())
			throw neural_network_exception("create_testers: empty group");
		if (!cuda_config)
			cuda_config = running_configuration_b200::get_current();
		fused_testers res;
		chain_description chain;
		res.io = describe_group(g, nodes, chain);
		const schema_node& head = nodes.at(g.members[0]);
		layer::const_ptr head_schema(new layer(head.params));
		if (g.kind == fused_single_layer)
		{
			res.objects.push_back(create_tester(head_schema, own_input_shapes(head, shapes), shape_of(shapes, head.name), cuda_config));
			return res;
		}
		layer_tester_b200::ptr h;
		switch (g.kind)
		{
		case fused_bn_act:
			h.reset(new fused_bn_act_tester_b200(chain));
			break;
		case fused_bn_add_relu_maxpool:
		case fused_bn_add_relu_avgpool:
			h.reset(new fused_pooled_tester_b200(chain, nodes.at(g.pool).params, g.kind == fused_bn_add_relu_avgpool));
			break;
		case fused_softmax_nll:
			h.reset(new fused_softmax_nll_tester_b200(nodes.at(g.loss).params.scale));
			break;
		default:
			throw neural_network_exception("create_testers: group kind " + std::to_string((int)g.kind) + " is a training pattern");
		}
		h->configure(input_shapes(res.io, nodes, shapes), shape_of(shapes, nodes.at(res.io.output_sources[0]).name), head_schema, cuda_config);
		res.objects.push_back(h);
		for (size_t k = 1; k < g.members.size(); ++k)
		{
			const schema_node& n = nodes.at(g.members[k]);
			layer_tester_b200::ptr fl(new fused_follower_tester_b200(follower_in_place(g, g.members[k])));
			fl->configure(own_input_shapes(n, shapes), shape_of(shapes, n.name), layer::const_ptr(new layer(n.params)), cuda_config);
			res.objects.push_back(fl);
		}
		return res;
	}

	fused_updaters layer_factory_b200::create_updaters(const fused_group& g, const std::vector<schema_node>& nodes,
		const std::map<std::string, layer_configuration_specific>& shapes, const std::vector<std::set<layer_action>>& actions,
		running_configuration_b200::const_ptr cuda_config) const
	{
		if (g.members.empty() || actions.size() != g.members.size())
			throw neural_network_exception("create_updaters: one action set per member expected");
		if (!cuda_config)
			cuda_config = running_configuration_b200::get_current();
		fused_updaters res;
		chain_description chain;
		res.io = describe_group(g, nodes, chain);
		const schema_node& head = nodes.at(g.members[0]);
		layer::const_ptr head_schema(new layer(head.params));
		if (g.kind == fused_single_layer)
		{
			res.objects.push_back(create_updater(head_schema, own_input_shapes(head, shapes), shape_of(shapes, head.name), actions[0], cuda_config));
			return res;
		}
		layer_updater_b200::ptr h;
		switch (g.kind)
		{
		case fused_bn_train_act:
			h = make_batch_norm_updater(chain.acts);
			break;
		case fused_softmax_nll:
			h.reset(new fused_softmax_nll_updater_b200(nodes.at(g.loss).params.scale));
			break;
		default:
			throw neural_network_exception("create_updaters: group kind " + std::to_string((int)g.kind) + " is an inference pattern");
		}
		h->configure(input_shapes(res.io, nodes, shapes), shape_of(shapes, nodes.at(res.io.output_sources[0]).name), head_schema, cuda_config, actions[0]);
		res.objects.push_back(h);
		for (size_t k = 1; k < g.members.size(); ++k)
		{
			const schema_node& n = nodes.at(g.members[k]);
			layer_updater_b200::ptr fl(new fused_follower_updater_b200(follower_in_place(g, g.members[k])));
			fl->configure(own_input_shapes(n, shapes), shape_of(shapes, n.name), layer::const_ptr(new layer(n.params)), cuda_config, actions[k]);
			res.objects.push_back(fl);
		}
		return res;
	}
}

// ---- flat driver: the objects of a whole textual schema ------------------------------------------------
// nnfh_net_create parses the schema (parse_schema), plans it (plan_fusion), infers every layer's output shape and
// creates the objects of every group through the factory, on the current device. The caller - the tests' and the
// benchmark's small scheduler - then asks nnfh_net_describe which object reads and writes what, and enqueues the
// objects through the nnfh_* calls that take a layer handle (nnfh_net_object).
using namespace nnf_b200;

namespace
{
	thread_local std::string g_net_error;

	struct net_object
	{
		detail::flat_handle handle;
		int group = 0;
		int node = 0;
		std::string role; // head, follower or single
		fused_io io;
	};

	struct net
	{
		std::vector<schema_node> nodes;
		std::map<std::string, layer_configuration_specific> shapes;
		std::vector<fused_group> plan;
		std::vector<std::unique_ptr<net_object>> objects;
		peer_directory::ptr peers;
	};

	std::set<layer_action> default_actions(const schema_node& n)
	{
		std::set<layer_action> a;
		a.insert(layer_action(layer_action::forward));
		const std::string& t = n.params.type_name;
		if (t == "BatchNorm")
			a.insert(layer_action(layer_action::backward_data_and_weights));
		else if (t == "Accuracy")
			;
		else if (t == "NegativeLogLikelihood" || t == "CrossEntropy")
			a.insert(layer_action(layer_action::backward_data, 0));
		else
		{
			for (size_t k = 0; k < n.inputs.size(); ++k)
				a.insert(layer_action(layer_action::backward_data, (int)k));
			if (t == "PReLU")
				a.insert(layer_action(layer_action::backward_weights));
		}
		return a;
	}

	const char * kKindNames[] = {"single", "bn_act", "bn_add_relu_maxpool", "bn_add_relu_avgpool", "bn_train_act", "softmax_nll"};
}

#define NNFH_API extern "C" __attribute__((visibility("default")))

NNFH_API const char * nnfh_net_last_error() { return g_net_error.c_str(); }

NNFH_API void * nnfh_peer_directory_create() { return new peer_directory::ptr(new peer_directory()); }
NNFH_API void nnfh_peer_directory_destroy(void * d) { delete static_cast<peer_directory::ptr *>(d); }
NNFH_API void nnfh_peer_directory_publish(void * d, const char * key, int device_pos, void * address)
{
	(*static_cast<peer_directory::ptr *>(d))->publish(key, device_pos, address);
}

// data_shapes: one data layer per line, "name feature_maps w h". peers: from nnfh_peer_directory_create, or null with one device.
NNFH_API void * nnfh_net_create(const char * spec, int training, const char * data_shapes, int device_pos, int device_count, void * peers)
{
	try
	{
		std::unique_ptr<net> n(new net());
		n->nodes = parse_schema(spec);
		n->plan = plan_fusion(n->nodes, training != 0);
		std::stringstream ds(data_shapes ? data_shapes : "");
		std::string name;
		unsigned int fm, w, h;
		while (ds >> name >> fm >> w >> h)
		{
			layer_configuration_specific c;
			c.feature_map_count = fm;
			c.dimension_sizes = {w, h};
			n->shapes[name] = c;
		}
		for (const schema_node& node : n->nodes)
		{
			std::vector<layer_configuration_specific> ins;
			for (const std::string& in : node.inputs)
			{
				if (!n->shapes.count(in))
					throw neural_network_exception("No shape known for input " + in + " of layer " + node.name);
				ins.push_back(n->shapes[in]);
			}
			if (ins.empty())
				throw neural_network_exception("Layer " + node.name + " has no inputs: give data layers in data_shapes, not in the schema");
			n->shapes[node.name] = get_output_layer_configuration_specific(node.params, ins);
		}
		int device = 0;
		if (cudaGetDevice(&device) != cudaSuccess)
		{
			cudaGetLastError();
			device = 0;
		}
		if (peers)
			n->peers = *static_cast<peer_directory::ptr *>(peers);
		running_configuration_b200::const_ptr config(new running_configuration_b200(device, device_pos, device_count, n->peers));
		for (size_t gi = 0; gi < n->plan.size(); ++gi)
		{
			const fused_group& g = n->plan[gi];
			std::vector<layer_tester_b200::ptr> testers;
			std::vector<layer_updater_b200::ptr> updaters;
			fused_io io;
			if (training)
			{
				std::vector<std::set<layer_action>> actions;
				for (int m : g.members)
					actions.push_back(default_actions(n->nodes[m]));
				fused_updaters u = layer_factory_b200::get_singleton().create_updaters(g, n->nodes, n->shapes, actions, config);
				updaters = u.objects;
				io = u.io;
			}
			else
			{
				fused_testers t = layer_factory_b200::get_singleton().create_testers(g, n->nodes, n->shapes, config);
				testers = t.objects;
				io = t.io;
			}
			for (size_t k = 0; k < g.members.size(); ++k)
			{
				std::unique_ptr<net_object> o(new net_object());
				o->group = (int)gi;
				o->node = g.members[k];
				o->role = g.kind == fused_single_layer ? "single" : k == 0 ? "head" : "follower";
				if (k == 0)
					o->io = io;
				o->handle.schema.reset(new layer(n->nodes[g.members[k]].params));
				if (training)
					o->handle.updater = updaters.at(k);
				else
					o->handle.tester = testers.at(k);
				n->objects.push_back(std::move(o));
			}
		}
		return n.release();
	}
	catch (const std::exception& e)
	{
		g_net_error = e.what();
		return nullptr;
	}
}

NNFH_API void nnfh_net_destroy(void * n) { delete static_cast<net *>(n); }

NNFH_API int nnfh_net_object_count(void * n) { return (int)static_cast<net *>(n)->objects.size(); }

// a layer handle for the nnfh_* calls; owned by the net
NNFH_API void * nnfh_net_object(void * n, int index)
{
	net& nt = *static_cast<net *>(n);
	return index >= 0 && index < (int)nt.objects.size() ? &nt.objects[index]->handle : nullptr;
}

// One object per line, in execution order:
//   "node=<name> type=<type> role=<head|follower|single> group=<i> kind=<kind> entry=<C-ABI call|-> shape=<fm>,<w>,<h>
//    inputs=<layer>:<input index>,... data=<layer>,... outputs=<layer>,... elided=<layer>,..."
// inputs / data / outputs / elided describe what the object itself takes: "-" for followers.
NNFH_API int nnfh_net_describe(void * n, char * out, size_t out_size)
{
	try
	{
		net& nt = *static_cast<net *>(n);
		std::stringstream res;
		for (const auto& o : nt.objects)
		{
			const fused_group& g = nt.plan[o->group];
			const schema_node& node = nt.nodes[o->node];
			const layer_configuration_specific& shape = nt.shapes[node.name];
			res << "node=" << node.name << " type=" << node.params.type_name << " role=" << o->role << " group=" << o->group << " kind=" << kKindNames[g.kind]
				<< " entry=" << (g.entry_point.empty() ? "-" : g.entry_point)
				<< " shape=" << shape.feature_map_count << "," << shape.dimension_sizes.at(0) << "," << (shape.dimension_sizes.size() > 1 ? shape.dimension_sizes[1] : 1);
			const bool runs = o->role != "follower";
			res << " inputs=";
			if (!runs || o->io.input_sources.empty())
				res << "-";
			else
				for (size_t k = 0; k < o->io.input_sources.size(); ++k)
					res << (k ? "," : "") << nt.nodes[o->io.input_sources[k].first].inputs.at(o->io.input_sources[k].second);
			auto names = [&](const char * key, const std::vector<int>& v, bool show)
			{
				res << " " << key << "=";
				if (!show || v.empty())
					res << "-";
				else
					for (size_t k = 0; k < v.size(); ++k)
						res << (k ? "," : "") << nt.nodes[v[k]].name;
			};
			names("data", o->io.data_sources, runs);
			names("outputs", o->io.output_sources, runs);
			names("elided", g.elided, runs);
			res << "\n";
		}
		const std::string text = res.str();
		if (text.size() + 1 > out_size)
			throw neural_network_exception("Result buffer too small");
		memcpy(out, text.c_str(), text.size() + 1);
		return 0;
	}
	catch (const std::exception& e)
	{
		g_net_error = e.what();
		return -1;
	}
}

// The buffer plan of an inference net (plan_forward_buffers with the objects' own get_input_index_layer_can_write answers):
// first line "buffers=<count> total_bytes_per_entry=<n>", then one line per layer, "node=<name> buffer=<index|-> in_place=<input|->
// bytes_per_entry=<n>".
NNFH_API int nnfh_net_buffer_plan(void * n, char * out, size_t out_size)
{
	try
	{
		net& nt = *static_cast<net *>(n);
		const int count = (int)nt.nodes.size();
		std::vector<int> can_write(count, -1);
		std::vector<size_t> bytes(count, 0);
		for (const auto& o : nt.objects)
		{
			if (!o->handle.tester)
				throw neural_network_exception("nnfh_net_buffer_plan: the plan covers inference nets (testers)");
			can_write[o->node] = o->handle.tester->get_input_index_layer_can_write();
		}
		for (int i = 0; i < count; ++i)
			bytes[i] = size_t(nt.shapes[nt.nodes[i].name].get_neuron_count()) * sizeof(float);
		const buffer_plan bp = plan_forward_buffers(nt.nodes, nt.plan, can_write, bytes);
		std::stringstream res;
		res << "buffers=" << bp.buffer_bytes_per_entry.size() << " total_bytes_per_entry=" << bp.total_bytes_per_entry << "\n";
		for (int i = 0; i < count; ++i)
		{
			res << "node=" << nt.nodes[i].name << " buffer=";
			if (bp.buffer_of_node[i] < 0) res << "-"; else res << bp.buffer_of_node[i];
			res << " in_place=";
			if (bp.written_in_place[i] < 0) res << "-"; else res << bp.written_in_place[i];
			res << " bytes_per_entry=" << bytes[i] << "\n";
		}
		const std::string text = res.str();
		if (text.size() + 1 > out_size)
			throw neural_network_exception("Result buffer too small");
		memcpy(out, text.c_str(), text.size() + 1);
		return 0;
	}
	catch (const std::exception& e)
	{
		g_net_error = e.what();
		return -1;
	}
}

// Lets `device` address the memory of `peer` (both directions are needed for a mailbox exchange: call it twice).
// Returns 0 when access is, or already was, enabled.
NNFH_API int nnfh_enable_peer_access(int device, int peer)
{
	int previous = 0;
	if (cudaGetDevice(&previous) != cudaSuccess)
		return -1;
	int ok = 0;
	if (cudaDeviceCanAccessPeer(&ok, device, peer) != cudaSuccess || !ok)
		return -1;
	cudaSetDevice(device);
	const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
	cudaGetLastError();
	cudaSetDevice(previous);
	return (e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled) ? 0 : -1;
}
