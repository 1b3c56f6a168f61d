// Implementation of the host-side layer objects (see nnf_layers.h) on top of the C ABI, plus a small
// flat driver interface (nnfh_*) through which the Python tests create these objects by type name
// and call their members with raw device pointers.
#include "nnf_layers_detail.h"

namespace nnf_b200
{
	using namespace detail;

	namespace
	{
		// ---- testers ---------------------------------------------------------------------------
		class batch_norm_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (data.size() != 4)
					throw neural_network_exception("BatchNorm expects 4 weight chunks: gamma, beta, mean, inverse sigma");
				check(nnf_bn_infer_act(stream_id, f(output_buffer), f(input_buffers[0]), f(data[0]), f(data[1]), f(data[2]), f(data[3]),
					nullptr, 1.0F, nullptr, 0, entry_count, output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			int get_input_index_layer_can_write() const override { return 0; }
		};

		class activation_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				const nnf_act a = make_act(*layer_schema, data.empty() ? nullptr : f(data[0]));
				check(nnf_act_fwd(stream_id, f(output_buffer), f(input_buffers[0]), &a, entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			int get_input_index_layer_can_write() const override { return 0; }
		};

		class add_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				std::vector<const float *> in;
				for (const auto& b : input_buffers)
					in.push_back(f(b));
				check(nnf_add_fwd(stream_id, f(output_buffer), in.data(), (int)in.size(), layer_schema->alpha, (int64_t)entry_count * output_elem_count_per_entry));
			}
			int get_input_index_layer_can_write() const override { return 0; }
		};

		class softmax_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				check(nnf_softmax_fwd(stream_id, f(output_buffer), f(input_buffers[0]), entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			int get_input_index_layer_can_write() const override { return 0; }
		};

		// average_subsampling_layer over the spatial dimensions (nnforge/cuda/average_subsampling_layer_tester_cuda.cu);
		// layer_schema->alpha is the effective alpha (the plain backend's default for spatial windows is 1)
		class average_subsampling_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				check(nnf_avgpool_fwd(stream_id, f(output_buffer), f(input_buffers[0]), entry_count, in.feature_map_count, in.dimension_sizes.at(1), in.dimension_sizes.at(0),
					(int)layer_schema->subsampling_sizes.at(0), (int)layer_schema->subsampling_sizes.at(1), layer_schema->alpha));
			}
		};

		// negative_log_likelihood_layer: inputs = predicted, actual[, scale mask]; output = one value per (entry, pixel)
		// (nnforge/cuda/negative_log_likelihood_layer_tester_cuda.cu)
		class negative_log_likelihood_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (input_buffers.size() < 2)
					throw neural_network_exception("negative_log_likelihood_layer needs the predicted and the actual values");
				check(nnf_nll_fwd(stream_id, f(output_buffer), f(input_buffers[0]), f(input_buffers[1]), input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr,
					layer_schema->scale, entry_count, input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map));
			}
		};

		// cross_entropy_layer: inputs = predicted, actual[, scale mask]; output = one value per (entry, pixel)
		// (nnforge/cuda/cross_entropy_layer_tester_cuda.cu). The plain tester takes the mask INSTEAD of the scale when a mask is
		// given (nnforge/plain/cross_entropy_layer_tester_plain.cpp:72-74): a scale of 1 reproduces it.
		class cross_entropy_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (input_buffers.size() < 2)
					throw neural_network_exception("cross_entropy_layer needs the predicted and the actual values");
				const bool masked = input_buffers.size() > 2;
				check(nnf_cross_entropy_fwd(stream_id, f(output_buffer), f(input_buffers[0]), f(input_buffers[1]), masked ? f(input_buffers[2]) : nullptr,
					masked ? 1.0F : layer_schema->scale, entry_count, input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map));
			}
		};

		// accuracy_layer: inputs = predicted, actual[, mask]; output = top_n + 1 planes per entry (nnforge/cuda/accuracy_layer_tester_cuda.cu)
		class accuracy_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (input_buffers.size() < 2)
					throw neural_network_exception("accuracy_layer needs the predicted and the actual values");
				check(nnf_accuracy_fwd(stream_id, f(output_buffer), f(input_buffers[0]), f(input_buffers[1]), input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr,
					(int)layer_schema->top_n, entry_count, input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map));
			}
		};

		class max_subsampling_layer_tester_b200 : public layer_tester_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				check(nnf_maxpool_fwd(stream_id, f(output_buffer), nullptr, f(input_buffers[0]), entry_count, in.feature_map_count, dim(in, 1), dim(in, 0), &pool));
			}
		protected:
			void tester_configured() override { pool = make_pool(*layer_schema, input_configuration_specific_list[0]); }
			nnf_pool pool;
		};

		// ---- updaters --------------------------------------------------------------------------
		class activation_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				const nnf_act a = make_act(*layer_schema, data.empty() ? nullptr : f(data[0]));
				check(nnf_act_fwd(stream_id, f(output_buffer), f(input_buffers[0]), &a, entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr output_errors_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_neurons_buffers, device_buffer::const_ptr output_neurons_buffer,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				const nnf_act a = make_act(*layer_schema, data.empty() ? nullptr : f(data[0]));
				const float * neurons = backward_uses_input(*layer_schema) ? f(input_neurons_buffers[0]) : f(output_neurons_buffer);
				check(nnf_act_bwd(stream_id, f(input_errors_buffer), f(output_errors_buffer), neurons, &a, entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map, add_update_to_destination ? 1 : 0));
			}
			void enqueue_backward_weights_propagation(cudaStream_t stream_id, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::ptr>& gradient, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_neurons_buffers, device_buffer::const_ptr output_errors_buffer,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr temporary_working_fixed_buffer, device_buffer::ptr,
				device_buffer::const_ptr, device_buffer::const_ptr, unsigned int entry_count) override
			{
				if (layer_schema->type_name != "PReLU")
					throw neural_network_exception("backward_weights requested from a layer without weights: " + layer_schema->type_name);
				check(nnf_prelu_bwd_weights(stream_id, f(gradient[0]), f(output_errors_buffer), f(input_neurons_buffers[0]), entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map,
					temporary_working_fixed_buffer ? static_cast<void *>(*temporary_working_fixed_buffer) : nullptr,
					temporary_working_fixed_buffer ? temporary_working_fixed_buffer->get_size() : 0));
			}
			std::pair<size_t, bool> get_temporary_working_fixed_buffer_size(const layer_action& action) const override
			{
				if (action.get_action_type() == layer_action::backward_weights)
					return std::make_pair(nnf_prelu_bwd_weights_workspace_bytes(1, output_configuration_specific.feature_map_count, output_elem_count_per_feature_map), false);
				return std::make_pair(size_t(0), false);
			}
			int get_input_index_layer_can_write(const layer_action&) const override { return 0; }
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return backward_uses_input(*layer_schema); }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return !backward_uses_input(*layer_schema); }
			bool is_backward_weights_dependent_on_input_buffer(unsigned int) const override { return true; }
		};

		class add_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				std::vector<const float *> in;
				for (const auto& b : input_buffers)
					in.push_back(f(b));
				check(nnf_add_fwd(stream_id, f(output_buffer), in.data(), (int)in.size(), layer_schema->alpha, (int64_t)entry_count * output_elem_count_per_entry));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr output_errors_buffer, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				check(nnf_add_bwd(stream_id, f(input_errors_buffer), f(output_errors_buffer), layer_schema->alpha,
					(int64_t)entry_count * output_elem_count_per_entry, add_update_to_destination ? 1 : 0));
			}
			int get_input_index_layer_can_write(const layer_action&) const override { return 0; }
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return false; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return false; }
		};

		class softmax_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				check(nnf_softmax_fwd(stream_id, f(output_buffer), f(input_buffers[0]), entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr output_errors_buffer, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr output_neurons_buffer,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				check(nnf_softmax_bwd(stream_id, f(input_errors_buffer), f(output_errors_buffer), f(output_neurons_buffer), entry_count,
					output_configuration_specific.feature_map_count, output_elem_count_per_feature_map, add_update_to_destination ? 1 : 0));
			}
			int get_input_index_layer_can_write(const layer_action& action) const override { return action.get_action_type() == layer_action::backward_data ? 0 : -1; }
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return false; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return true; }
		};

		class average_subsampling_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				check(nnf_avgpool_fwd(stream_id, f(output_buffer), f(input_buffers[0]), entry_count, in.feature_map_count, in.dimension_sizes.at(1), in.dimension_sizes.at(0),
					(int)layer_schema->subsampling_sizes.at(0), (int)layer_schema->subsampling_sizes.at(1), layer_schema->alpha));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr output_errors_buffer, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				check(nnf_avgpool_bwd(stream_id, f(input_errors_buffer), f(output_errors_buffer), entry_count, in.feature_map_count, in.dimension_sizes.at(1), in.dimension_sizes.at(0),
					(int)layer_schema->subsampling_sizes.at(0), (int)layer_schema->subsampling_sizes.at(1), layer_schema->alpha, add_update_to_destination ? 1 : 0));
			}
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return false; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return false; }
		};

		// (nnforge/cuda/negative_log_likelihood_layer_updater_cuda.cu; the layer is a loss: backward reads no output errors)
		class negative_log_likelihood_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (input_buffers.size() < 2)
					throw neural_network_exception("negative_log_likelihood_layer needs the predicted and the actual values");
				check(nnf_nll_fwd(stream_id, f(output_buffer), f(input_buffers[0]), f(input_buffers[1]), input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr,
					layer_schema->scale, entry_count, input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int input_index, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>& input_neurons_buffers, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				if (input_index != 0)
					throw neural_network_exception("negative_log_likelihood_layer_updater cannot do backward propagation for targets or the scale mask");
				check(nnf_nll_bwd(stream_id, f(input_errors_buffer), f(input_neurons_buffers.at(0)), f(input_neurons_buffers.at(1)),
					input_neurons_buffers.size() > 2 ? f(input_neurons_buffers[2]) : nullptr, layer_schema->scale, entry_count,
					input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map, add_update_to_destination ? 1 : 0));
			}
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return true; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return false; }
		};

		// (nnforge/cuda/cross_entropy_layer_updater_cuda.cu; the layer is a loss: backward reads no output errors)
		class cross_entropy_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (input_buffers.size() < 2)
					throw neural_network_exception("cross_entropy_layer needs the predicted and the actual values");
				check(nnf_cross_entropy_fwd(stream_id, f(output_buffer), f(input_buffers[0]), f(input_buffers[1]), input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr,
					layer_schema->scale, entry_count, input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int input_index, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>& input_neurons_buffers, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				if (input_index == 1)
					throw neural_network_exception("cross_entropy_layer_updater cannot do backward propagation for targets");
				if (input_index == 2)
					throw neural_network_exception("cross_entropy_layer_updater cannot do backward propagation for scale mask");
				check(nnf_cross_entropy_bwd(stream_id, f(input_errors_buffer), f(input_neurons_buffers.at(0)), f(input_neurons_buffers.at(1)),
					input_neurons_buffers.size() > 2 ? f(input_neurons_buffers[2]) : nullptr, layer_schema->scale, entry_count,
					input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map, add_update_to_destination ? 1 : 0));
			}
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return true; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return false; }
		};

		// forward only, like the stock updater (nnforge/cuda/accuracy_layer_updater_cuda.cu)
		class accuracy_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, unsigned int entry_count) override
			{
				if (input_buffers.size() < 2)
					throw neural_network_exception("accuracy_layer needs the predicted and the actual values");
				check(nnf_accuracy_fwd(stream_id, f(output_buffer), f(input_buffers[0]), f(input_buffers[1]), input_buffers.size() > 2 ? f(input_buffers[2]) : nullptr,
					(int)layer_schema->top_n, entry_count, input_configuration_specific_list[0].feature_map_count, output_elem_count_per_feature_map));
			}
		};

		class max_subsampling_layer_updater_b200 : public layer_updater_b200
		{
		public:
			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr, device_buffer::ptr, device_buffer::ptr, device_buffer::ptr temporary_per_entry_buffer, unsigned int entry_count) override
			{
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				check(nnf_maxpool_fwd(stream_id, f(output_buffer), temporary_per_entry_buffer ? static_cast<unsigned int *>(*temporary_per_entry_buffer) : nullptr,
					f(input_buffers[0]), entry_count, in.feature_map_count, dim(in, 1), dim(in, 0), &pool));
			}
			void enqueue_backward_data_propagation(cudaStream_t stream_id, unsigned int, device_buffer::ptr input_errors_buffer,
				device_buffer::const_ptr output_errors_buffer, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr,
				const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr,
				device_buffer::const_ptr temporary_per_entry_buffer, bool add_update_to_destination, unsigned int entry_count) override
			{
				if (!temporary_per_entry_buffer)
					throw neural_network_exception("MaxSubsampling backward needs the argmax buffer written by its forward action");
				const layer_configuration_specific& in = input_configuration_specific_list[0];
				check(nnf_maxpool_bwd(stream_id, f(input_errors_buffer), f(output_errors_buffer), static_cast<const unsigned int *>(*temporary_per_entry_buffer),
					entry_count, in.feature_map_count, dim(in, 1), dim(in, 0), &pool, add_update_to_destination ? 1 : 0));
			}
			// absolute input offsets as unsigned int, the plain backend's format (max_subsampling_layer_updater_plain.cpp:256-264)
			size_t get_temporary_per_entry_buffer_size() const override
			{
				return actions.count(layer_action(layer_action::backward_data, 0)) ? size_t(output_elem_count_per_entry) * sizeof(unsigned int) : 0;
			}
			bool is_backward_data_dependent_on_input_buffer(unsigned int, unsigned int) const override { return false; }
			bool is_backward_data_dependent_on_output_buffer(unsigned int) const override { return false; }
		protected:
			void updater_configured() override { pool = make_pool(*layer_schema, input_configuration_specific_list[0]); }
			nnf_pool pool;
		};

		// Training-mode batch norm, alone or as the head of a fused BatchNorm -> activations group (the followers'
		// parameters are then in `followers`, their weight chunks behind the batch norm's four in data / gradient).
		// temporary_fixed_buffer = {mean, inverse std-dev} (2*C floats, as stock);
		// temporary_working_fixed_buffer = the kernels' workspace followed by 2*C (forward) or 3*C (backward) floats of sums.
		// With more than one device sharing the batch (cuda_config->device_count > 1) the statistics are those of the
		// whole batch: the object owns a mailbox (get_persistent_working_data), publishes its address in
		// cuda_config->peers under the layer's instance name and runs the batch-sharded single-launch entry points;
		// every device must enqueue the same action with the same entry_count.
		class batch_norm_layer_updater_b200 : public layer_updater_b200
		{
		public:
			explicit batch_norm_layer_updater_b200(const std::vector<layer>& followers = std::vector<layer>()) : followers(followers) {}

			void enqueue_forward_propagation(cudaStream_t stream_id, device_buffer::ptr output_buffer, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_buffers, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr temporary_working_fixed_buffer, device_buffer::ptr, device_buffer::ptr temporary_fixed_buffer, device_buffer::ptr,
				unsigned int entry_count) override
			{
				if (data.size() != chunk_count())
					throw neural_network_exception("BatchNorm expects " + std::to_string(chunk_count()) + " weight chunks: gamma, beta, mean, inverse sigma and one slope chunk per fused PReLU");
				const unsigned int c = output_configuration_specific.feature_map_count;
				char * ws = working(temporary_working_fixed_buffer, 2);
				float * sums = reinterpret_cast<float *>(ws + workspace_bytes());
				const std::vector<nnf_act> acts = make_acts(data);
				if (sharded())
				{
					const std::vector<void *> boxes = mailboxes();
					check(nnf_bn_train_fwd_sharded(stream_id, f(output_buffer), f(temporary_fixed_buffer), sums, f(input_buffers[0]), f(data[0]), f(data[1]),
						layer_schema->epsilon, acts.data(), (int)acts.size(), entry_count, c, output_elem_count_per_feature_map, count_total(entry_count),
						ws, workspace_bytes(), boxes.data(), cuda_config->device_pos, cuda_config->device_count, ++seq));
				}
				else
					check(nnf_bn_train_fwd(stream_id, f(output_buffer), f(temporary_fixed_buffer), sums, f(input_buffers[0]), f(data[0]), f(data[1]),
						layer_schema->epsilon, acts.empty() ? nullptr : acts.data(), (int)acts.size(), entry_count, c, output_elem_count_per_feature_map, ws, workspace_bytes()));
			}
			void enqueue_backward_data_and_weights_propagation(cudaStream_t stream_id, const std::vector<device_buffer::ptr> input_errors_buffers,
				device_buffer::const_ptr output_errors_buffer, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::ptr>& gradient,
				const std::vector<device_buffer::const_ptr>& data, const std::vector<device_buffer::const_ptr>&,
				const std::vector<device_buffer::const_ptr>& input_neurons_buffers, device_buffer::const_ptr, const std::vector<device_buffer::const_ptr>&,
				device_buffer::ptr temporary_working_fixed_buffer, device_buffer::ptr, device_buffer::const_ptr temporary_fixed_buffer, device_buffer::const_ptr,
				bool add_update_to_destination, unsigned int entry_count) override
			{
				if (gradient.size() != chunk_count() || data.size() != chunk_count())
					throw neural_network_exception("BatchNorm expects " + std::to_string(chunk_count()) + " weight chunks and as many gradient chunks");
				const unsigned int c = output_configuration_specific.feature_map_count;
				char * ws = working(temporary_working_fixed_buffer, 3);
				float * bsums = reinterpret_cast<float *>(ws + workspace_bytes());
				const std::vector<nnf_act> acts = make_acts(data);
				float * grad_slope = nullptr;
				for (size_t k = 0, chunk = 4; k < followers.size(); ++k)
					if (followers[k].type_name == "PReLU")
						grad_slope = f(gradient[chunk++]);
				// gradient[0..3] = gamma, beta, mean, inverse sigma; running statistics are trained through the
				// pseudo-gradients of batch_norm_layer_updater_cuda.cu:167-182
				if (sharded())
				{
					if (add_update_to_destination)
						throw neural_network_exception("BatchNorm: add_update_to_destination is not available when the batch is shared by several devices");
					const std::vector<void *> boxes = mailboxes();
					check(nnf_bn_train_bwd_sharded(stream_id, f(input_errors_buffers[0]), bsums, f(output_errors_buffer), f(input_neurons_buffers[0]), f(data[0]), f(data[1]),
						f(temporary_fixed_buffer), acts.data(), (int)acts.size(), f(gradient[0]), f(gradient[1]), f(gradient[2]), f(gradient[3]), grad_slope,
						f(data[2]), f(data[3]), (float)entry_count, entry_count, c, output_elem_count_per_feature_map, count_total(entry_count),
						ws, workspace_bytes(), boxes.data(), cuda_config->device_pos, cuda_config->device_count, ++seq));
				}
				else
					check(nnf_bn_train_bwd(stream_id, f(input_errors_buffers[0]), bsums, f(output_errors_buffer), f(input_neurons_buffers[0]), f(data[0]), f(data[1]),
						f(temporary_fixed_buffer), acts.empty() ? nullptr : acts.data(), (int)acts.size(), f(gradient[0]), f(gradient[1]), f(gradient[2]), f(gradient[3]),
						grad_slope, f(data[2]), f(data[3]), (float)entry_count, entry_count, c, output_elem_count_per_feature_map, add_update_to_destination ? 1 : 0,
						ws, workspace_bytes()));
			}
			std::vector<device_buffer::const_ptr> get_persistent_working_data() const override
			{
				return mailbox ? std::vector<device_buffer::const_ptr>(1, mailbox) : std::vector<device_buffer::const_ptr>();
			}
			std::pair<size_t, bool> get_temporary_working_fixed_buffer_size(const layer_action& action) const override
			{
				const size_t c = output_configuration_specific.feature_map_count;
				if (action.get_action_type() == layer_action::forward)
					return std::make_pair(workspace_bytes() + 2 * c * sizeof(float), false);
				if (action.get_action_type() == layer_action::backward_data_and_weights)
					return std::make_pair(workspace_bytes() + 3 * c * sizeof(float), false);
				return std::make_pair(size_t(0), false);
			}
			size_t get_temporary_fixed_buffer_size() const override { return size_t(output_configuration_specific.feature_map_count) * 2 * sizeof(float); }
			int get_input_index_layer_can_write(const layer_action& action) const override { return action.get_action_type() == layer_action::backward_data_and_weights ? 0 : -1; }
			// backward recomputes the chain from x and the saved statistics: the group's output is not read
			bool is_backward_data_and_weights_dependent_on_input_buffer(unsigned int) const override { return true; }
			bool is_backward_data_and_weights_dependent_on_output_buffer() const override { return false; }
			bool is_backward_data_and_weights_dependent_on_temporary_fixed_buffer() const override { return true; }
			bool is_backward_data_and_weights_dependent_on_temporary_per_entry_buffer() const override { return false; }
		protected:
			void updater_configured() override
			{
				if (followers.size() > 2)
					throw neural_network_exception("BatchNorm can carry at most two fused activation layers");
				if (!sharded())
					return;
				if (!cuda_config->peers)
					throw neural_network_exception("BatchNorm: several devices share the batch but the running configuration has no peer directory");
				if (layer_schema->instance_name.empty())
					throw neural_network_exception("BatchNorm: several devices share the batch: the layer needs an instance name to publish its mailbox under");
				const size_t bytes = nnf_bn_train_mailbox_bytes(output_configuration_specific.feature_map_count);
				if (void * given = cuda_config->peers->find(layer_schema->instance_name, cuda_config->device_pos))
				{
					// one process per GPU: the process made a mailbox the others can map, and cleared it
					mailbox.reset(new device_buffer(given, bytes));
					return;
				}
				mailbox.reset(new device_buffer(bytes));
				if (cudaMemset(static_cast<void *>(*mailbox), 0, bytes) != cudaSuccess)
					throw neural_network_exception("BatchNorm: clearing the mailbox failed");
				cuda_config->peers->publish(layer_schema->instance_name, cuda_config->device_pos, static_cast<void *>(*mailbox));
			}
		private:
			bool sharded() const { return cuda_config && cuda_config->device_count > 1; }
			size_t chunk_count() const
			{
				size_t n = 4;
				for (const layer& l : followers)
					n += l.type_name == "PReLU";
				return n;
			}
			std::vector<nnf_act> make_acts(const std::vector<device_buffer::const_ptr>& data) const
			{
				std::vector<nnf_act> acts;
				size_t chunk = 4;
				for (const layer& l : followers)
					acts.push_back(make_act(l, l.type_name == "PReLU" ? f(data[chunk++]) : nullptr));
				return acts;
			}
			std::vector<void *> mailboxes() const { return cuda_config->peers->lookup(layer_schema->instance_name, cuda_config->device_count); }
			double count_total(unsigned int entry_count) const
			{
				return (double)entry_count * (double)cuda_config->device_count * (double)output_elem_count_per_feature_map;
			}
			size_t workspace_bytes() const { return nnf_bn_train_workspace_bytes(1, output_configuration_specific.feature_map_count, output_elem_count_per_feature_map); }
			char * working(const device_buffer::ptr& b, int sums) const
			{
				const size_t need = workspace_bytes() + size_t(sums) * output_configuration_specific.feature_map_count * sizeof(float);
				if (!b || b->get_size() < need)
					throw neural_network_exception("BatchNorm: temporary_working_fixed_buffer is missing or smaller than get_temporary_working_fixed_buffer_size()");
				return static_cast<char *>(static_cast<void *>(*b));
			}
			std::vector<layer> followers;
			device_buffer::ptr mailbox;
			uint32_t seq = 0;
		};
	}

	namespace detail
	{
		layer_updater_b200::ptr make_batch_norm_updater(const std::vector<layer>& followers)
		{
			return layer_updater_b200::ptr(new batch_norm_layer_updater_b200(followers));
		}
	}

	// ---- plumbing types ---------------------------------------------------------------------------
	namespace
	{
		void cuda_check(cudaError_t e, const char * what)
		{
			if (e != cudaSuccess)
				throw neural_network_exception(std::string(what) + ": " + cudaGetErrorString(e));
		}
	}

	device_buffer::device_buffer(size_t bytes) : p(nullptr), bytes(bytes), owned(true)
	{
		cuda_check(cudaMalloc(&p, bytes > 0 ? bytes : 1), "cudaMalloc");
	}

	device_buffer::~device_buffer()
	{
		if (owned && p)
			cudaFree(p);
	}

	void peer_directory::publish(const std::string& key, int device_pos, void * address)
	{
		std::lock_guard<std::mutex> lock(m);
		entries[key][device_pos] = address;
	}

	void * peer_directory::find(const std::string& key, int device_pos) const
	{
		std::lock_guard<std::mutex> lock(m);
		auto it = entries.find(key);
		if (it == entries.end() || !it->second.count(device_pos))
			return nullptr;
		return it->second.at(device_pos);
	}

	std::vector<void *> peer_directory::lookup(const std::string& key, int device_count) const
	{
		std::lock_guard<std::mutex> lock(m);
		std::vector<void *> res;
		auto it = entries.find(key);
		for (int pos = 0; pos < device_count; ++pos)
		{
			if (it == entries.end() || !it->second.count(pos))
				throw neural_network_exception("peer_directory: no address published for " + key + " by device position " + std::to_string(pos));
			res.push_back(it->second.at(pos));
		}
		return res;
	}

	running_configuration_b200::running_configuration_b200(int device_id, int device_pos, int device_count, peer_directory::ptr peers)
		: device_id(device_id), device_pos(device_pos), device_count(device_count), peers(peers)
	{
		if (device_count < 1 || device_pos < 0 || device_pos >= device_count)
			throw neural_network_exception("running_configuration_b200: device position outside the device count");
		// without a device (build checks, host-logic tests) the library answers with its built-in figures
		int previous = 0;
		const bool have_device = cudaGetDevice(&previous) == cudaSuccess;
		if (have_device)
			cuda_check(cudaSetDevice(device_id), "cudaSetDevice");
		else
			cudaGetLastError();
		nnf_running_configuration rc;
		const int status = nnf_get_running_configuration(&rc);
		if (have_device)
			cudaSetDevice(previous);
		check(status);
		compute_capability_major = rc.compute_capability_major;
		compute_capability_minor = rc.compute_capability_minor;
		multiprocessor_count = rc.multiprocessor_count;
		max_threads_per_multiprocessor = rc.max_threads_per_multiprocessor;
		smem_per_block = (size_t)rc.max_shared_memory_per_block_optin;
		smem_per_multiprocessor = (size_t)rc.max_shared_memory_per_multiprocessor;
		l2_cache_size = rc.l2_cache_size;
		max_registers_per_multiprocessor = rc.max_registers_per_multiprocessor;
	}

	running_configuration_b200::const_ptr running_configuration_b200::get_current()
	{
		static std::mutex m;
		static std::map<int, const_ptr> cache;
		int device = 0;
		if (cudaGetDevice(&device) != cudaSuccess)
		{
			cudaGetLastError();
			device = 0;
		}
		std::lock_guard<std::mutex> lock(m);
		auto it = cache.find(device);
		if (it == cache.end())
			it = cache.insert(std::make_pair(device, const_ptr(new running_configuration_b200(device)))).first;
		return it->second;
	}

	void running_configuration_b200::set_device() const
	{
		cuda_check(cudaSetDevice(device_id), "cudaSetDevice");
	}

	void layer_tester_b200::configure(const std::vector<layer_configuration_specific>& in, const layer_configuration_specific& out, layer::const_ptr schema,
		running_configuration_b200::const_ptr config)
	{
		layer_schema = schema;
		cuda_config = config;
		input_configuration_specific_list = in;
		output_configuration_specific = out;
		output_elem_count_per_entry = out.get_neuron_count();
		output_elem_count_per_feature_map = out.get_neuron_count_per_feature_map();
		tester_configured();
	}

	void layer_updater_b200::configure(const std::vector<layer_configuration_specific>& in, const layer_configuration_specific& out, layer::const_ptr schema,
		running_configuration_b200::const_ptr config, const std::set<layer_action>& acts)
	{
		layer_schema = schema;
		cuda_config = config;
		input_configuration_specific_list = in;
		output_configuration_specific = out;
		output_elem_count_per_entry = out.get_neuron_count();
		output_elem_count_per_feature_map = out.get_neuron_count_per_feature_map();
		actions = acts;
		updater_configured();
	}

	void layer_tester_b200::enqueue_forward_propagation(cudaStream_t stream_id, const std::vector<device_buffer::ptr>& output_buffers,
		const std::vector<device_buffer::const_ptr>& schema_data, const std::vector<device_buffer::const_ptr>& data,
		const std::vector<device_buffer::const_ptr>& data_custom, const std::vector<device_buffer::const_ptr>& input_buffers,
		const std::vector<device_buffer::const_ptr>& persistent_working_data, device_buffer::ptr temporary_working_fixed_buffer,
		device_buffer::ptr temporary_working_per_entry_buffer, unsigned int entry_count)
	{
		if (output_buffers.size() != 1)
			throw neural_network_exception("layer " + layer_schema->type_name + " writes one output, " + std::to_string(output_buffers.size()) + " output buffers given");
		enqueue_forward_propagation(stream_id, output_buffers[0], schema_data, data, data_custom, input_buffers, persistent_working_data,
			temporary_working_fixed_buffer, temporary_working_per_entry_buffer, entry_count);
	}

	void layer_updater_b200::enqueue_forward_propagation(cudaStream_t stream_id, const std::vector<device_buffer::ptr>& output_buffers,
		const std::vector<device_buffer::const_ptr>& schema_data, const std::vector<device_buffer::const_ptr>& data,
		const std::vector<device_buffer::const_ptr>& data_custom, const std::vector<device_buffer::const_ptr>& input_buffers,
		const std::vector<device_buffer::const_ptr>& persistent_working_data, device_buffer::ptr temporary_working_fixed_buffer,
		device_buffer::ptr temporary_working_per_entry_buffer, device_buffer::ptr temporary_fixed_buffer, device_buffer::ptr temporary_per_entry_buffer,
		unsigned int entry_count)
	{
		if (output_buffers.size() != 1)
			throw neural_network_exception("layer " + layer_schema->type_name + " writes one output, " + std::to_string(output_buffers.size()) + " output buffers given");
		enqueue_forward_propagation(stream_id, output_buffers[0], schema_data, data, data_custom, input_buffers, persistent_working_data,
			temporary_working_fixed_buffer, temporary_working_per_entry_buffer, temporary_fixed_buffer, temporary_per_entry_buffer, entry_count);
	}

	namespace
	{
		template<class T, class P>
		std::vector<P> upload(const std::vector<std::vector<T>>& host)
		{
			std::vector<P> res;
			for (const std::vector<T>& part : host)
			{
				device_buffer::ptr b(new device_buffer(part.size() * sizeof(T)));
				if (!part.empty())
					cuda_check(cudaMemcpy(static_cast<void *>(*b), part.data(), part.size() * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
				res.push_back(b);
			}
			return res;
		}
	}

	std::vector<device_buffer::const_ptr> layer_tester_b200::get_data(layer_data::const_ptr host_data) const
	{
		return upload<float, device_buffer::const_ptr>(*host_data);
	}

	std::vector<device_buffer::const_ptr> layer_tester_b200::set_get_data_custom(layer_data_custom::const_ptr host_data)
	{
		notify_data_custom(host_data);
		return upload<int, device_buffer::const_ptr>(*host_data);
	}

	std::vector<device_buffer::ptr> layer_updater_b200::get_data(layer_data::const_ptr host_data) const
	{
		return upload<float, device_buffer::ptr>(*host_data);
	}

	std::vector<device_buffer::const_ptr> layer_updater_b200::set_get_data_custom(layer_data_custom::const_ptr host_data)
	{
		notify_data_custom(host_data);
		return upload<int, device_buffer::const_ptr>(*host_data);
	}

	void layer_updater_b200::get_data_from_device(const std::vector<device_buffer::ptr>& device_data, layer_data::ptr host_data) const
	{
		if (device_data.size() != host_data->size())
			throw neural_network_exception("get_data_from_device: chunk counts differ");
		for (size_t part_id = 0; part_id < host_data->size(); ++part_id)
		{
			std::vector<float>& part = (*host_data)[part_id];
			if (!part.empty())
				cuda_check(cudaMemcpy(part.data(), static_cast<const void *>(*device_data[part_id]), part.size() * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy");
		}
	}

	// Defaults of the reference base class: an action the layer does not implement is an error
	// (nnforge/cuda/layer_updater_cuda.cpp throws "... is not implemented").
	void layer_updater_b200::enqueue_backward_data_propagation(cudaStream_t, unsigned int, device_buffer::ptr, device_buffer::const_ptr,
		const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&,
		const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr, const std::vector<device_buffer::const_ptr>&, device_buffer::ptr,
		device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr, bool, unsigned int)
	{
		throw neural_network_exception("enqueue_backward_data_propagation is not implemented for layer " + layer_schema->type_name);
	}

	void layer_updater_b200::enqueue_backward_weights_propagation(cudaStream_t, const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::ptr>&,
		const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr,
		const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr, unsigned int)
	{
		throw neural_network_exception("enqueue_backward_weights_propagation is not implemented for layer " + layer_schema->type_name);
	}

	void layer_updater_b200::enqueue_backward_data_and_weights_propagation(cudaStream_t, const std::vector<device_buffer::ptr>, device_buffer::const_ptr,
		const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::ptr>&, const std::vector<device_buffer::const_ptr>&,
		const std::vector<device_buffer::const_ptr>&, const std::vector<device_buffer::const_ptr>&, device_buffer::const_ptr,
		const std::vector<device_buffer::const_ptr>&, device_buffer::ptr, device_buffer::ptr, device_buffer::const_ptr, device_buffer::const_ptr, bool, unsigned int)
	{
		throw neural_network_exception("enqueue_backward_data_and_weights_propagation is not implemented for layer " + layer_schema->type_name);
	}

	layer_factory_b200& layer_factory_b200::get_singleton()
	{
		static layer_factory_b200 instance;
		return instance;
	}

	std::vector<std::string> layer_factory_b200::get_type_names() const
	{
		return {"BatchNorm", "ReLU", "PReLU", "ELU", "TanH", "Sigmoid", "Softmax", "Add", "MaxSubsampling", "NegativeLogLikelihood", "CrossEntropy", "Accuracy", "AverageSubsampling"};
	}

	layer_tester_b200::ptr layer_factory_b200::create_tester(layer::const_ptr l, const std::vector<layer_configuration_specific>& in,
		const layer_configuration_specific& out, running_configuration_b200::const_ptr cuda_config) const
	{
		layer_tester_b200::ptr t;
		const std::string& n = l->type_name;
		if (n == "BatchNorm") t.reset(new batch_norm_layer_tester_b200());
		else if (is_activation(n)) t.reset(new activation_layer_tester_b200());
		else if (n == "Add") t.reset(new add_layer_tester_b200());
		else if (n == "Softmax") t.reset(new softmax_layer_tester_b200());
		else if (n == "NegativeLogLikelihood") t.reset(new negative_log_likelihood_layer_tester_b200());
		else if (n == "CrossEntropy") t.reset(new cross_entropy_layer_tester_b200());
		else if (n == "Accuracy") t.reset(new accuracy_layer_tester_b200());
		else if (n == "AverageSubsampling") t.reset(new average_subsampling_layer_tester_b200());
		else if (n == "MaxSubsampling") t.reset(new max_subsampling_layer_tester_b200());
		else throw neural_network_exception("No layer tester is registered with id " + n);
		t->configure(in, out, l, cuda_config ? cuda_config : running_configuration_b200::get_current());
		return t;
	}

	layer_updater_b200::ptr layer_factory_b200::create_updater(layer::const_ptr l, const std::vector<layer_configuration_specific>& in,
		const layer_configuration_specific& out, const std::set<layer_action>& actions, running_configuration_b200::const_ptr cuda_config) const
	{
		layer_updater_b200::ptr u;
		const std::string& n = l->type_name;
		if (n == "BatchNorm") u.reset(new batch_norm_layer_updater_b200());
		else if (is_activation(n)) u.reset(new activation_layer_updater_b200());
		else if (n == "Add") u.reset(new add_layer_updater_b200());
		else if (n == "Softmax") u.reset(new softmax_layer_updater_b200());
		else if (n == "NegativeLogLikelihood") u.reset(new negative_log_likelihood_layer_updater_b200());
		else if (n == "CrossEntropy") u.reset(new cross_entropy_layer_updater_b200());
		else if (n == "Accuracy") u.reset(new accuracy_layer_updater_b200());
		else if (n == "AverageSubsampling") u.reset(new average_subsampling_layer_updater_b200());
		else if (n == "MaxSubsampling") u.reset(new max_subsampling_layer_updater_b200());
		else throw neural_network_exception("No layer updater is registered with id " + n);
		u->configure(in, out, l, cuda_config ? cuda_config : running_configuration_b200::get_current(), actions);
		return u;
	}

	layer_configuration_specific get_output_layer_configuration_specific(const layer& l, const std::vector<layer_configuration_specific>& inputs)
	{
		layer_configuration_specific res = inputs.at(0);
		if (l.type_name == "NegativeLogLikelihood" || l.type_name == "CrossEntropy")
			res.feature_map_count = 1; // negative_log_likelihood_layer.cpp:66, cross_entropy_layer.cpp:62
		if (l.type_name == "Accuracy")
			res.feature_map_count = l.top_n + 1; // accuracy_layer.cpp:62
		if (l.type_name == "AverageSubsampling")
			for (size_t i = 0; i < res.dimension_sizes.size(); ++i)
			{
				const unsigned int win = l.subsampling_sizes.at(i);
				if (win == 0 || inputs[0].dimension_sizes[i] % win != 0)
					throw neural_network_exception("Input configuration size of dimension " + std::to_string(i) + " is not evenly divisible by the subsampling size");
				res.dimension_sizes[i] = inputs[0].dimension_sizes[i] / win;
			}
		if (l.type_name == "MaxSubsampling")
		{
			const nnf_pool p = make_pool(l, inputs[0]);
			for (size_t i = 0; i < res.dimension_sizes.size(); ++i)
			{
				const int64_t o = nnf_pool_out_size(inputs[0].dimension_sizes[i], i == 0 ? p.win_w : p.win_h, i == 0 ? p.stride_w : p.stride_h, i == 0 ? p.round_up_w : p.round_up_h);
				if (o <= 0)
					throw neural_network_exception("Input configuration size of dimension " + std::to_string(i) + " produces 0 output size");
				res.dimension_sizes[i] = (unsigned int)o;
			}
		}
		return res;
	}

	void enqueue_apply_gradient(
		cudaStream_t stream_id,
		const std::vector<std::vector<device_buffer::ptr>>& data,
		const std::vector<std::vector<device_buffer::ptr>>& gradient,
		const std::vector<std::vector<device_buffer::ptr>>& prev_upd,
		const std::vector<std::vector<device_buffer::ptr>>& prev_upd2,
		const std::vector<std::vector<float>>& learning_rates,
		const std::vector<std::vector<device_buffer::ptr>>& update_accum_buffers,
		const std::vector<std::set<unsigned int>>& weight_decay_part_ids,
		float gradient_normalizer,
		float weight_decay,
		training_momentum momentum,
		unsigned int iteration_id)
	{
		const size_t layers = data.size();
		if (gradient.size() != layers || learning_rates.size() != layers || weight_decay_part_ids.size() != layers
			|| (momentum.is_momentum_data() && prev_upd.size() != layers) || (momentum.is_momentum_data2() && prev_upd2.size() != layers)
			|| (!update_accum_buffers.empty() && update_accum_buffers.size() != layers))
			throw neural_network_exception("enqueue_apply_gradient: the per-layer lists differ in length");
		std::vector<nnf_opt_part> parts;
		for (size_t l = 0; l < layers; ++l)
		{
			const size_t n = data[l].size();
			if (gradient[l].size() != n || learning_rates[l].size() != n || (momentum.is_momentum_data() && prev_upd[l].size() != n)
				|| (momentum.is_momentum_data2() && prev_upd2[l].size() != n))
				throw neural_network_exception("enqueue_apply_gradient: the chunk lists of a layer differ in length");
			const bool accum = !update_accum_buffers.empty() && !update_accum_buffers[l].empty();
			if (accum && update_accum_buffers[l].size() != n)
				throw neural_network_exception("enqueue_apply_gradient: one update accumulator per chunk expected");
			for (size_t part_id = 0; part_id < n; ++part_id)
			{
				nnf_opt_part p;
				p.data = *data[l][part_id];
				p.gradient = *gradient[l][part_id];
				p.prev_upd = momentum.is_momentum_data() ? (float *)*prev_upd[l][part_id] : nullptr;
				p.prev_upd2 = momentum.is_momentum_data2() ? (float *)*prev_upd2[l][part_id] : nullptr;
				p.update_accum = accum ? static_cast<double *>((void *)*update_accum_buffers[l][part_id]) : nullptr;
				p.learning_rate = learning_rates[l][part_id];
				p.weight_decay = weight_decay_part_ids[l].count((unsigned int)part_id) ? weight_decay : 0.0F;
				p.elem_count = (int64_t)(data[l][part_id]->get_size() / sizeof(float));
				parts.push_back(p);
			}
		}
		check(nnf_apply_gradient(stream_id, parts.data(), (int)parts.size(), (int)momentum.type, momentum.momentum_val, momentum.momentum_val2,
			gradient_normalizer, iteration_id));
	}
}

// ---- flat driver interface for tests (ctypes) ----------------------------------------------------
// Objects are created by type name through the factory; every call takes raw device pointers, wraps
// them in non-owning buffers and forwards to the C++ member with the reference's argument order.
// Return 0 on success; on an exception -1, with the text available from nnfh_last_error().
using namespace nnf_b200;

namespace
{
	thread_local std::string g_error;

	typedef nnf_b200::detail::flat_handle handle;

	device_buffer::ptr buf(void * p, size_t bytes = size_t(1) << 40) { return p ? device_buffer::ptr(new device_buffer(p, bytes)) : device_buffer::ptr(); }
	device_buffer::const_ptr cbuf(const void * p) { return p ? device_buffer::const_ptr(new device_buffer(const_cast<void *>(p), size_t(1) << 40)) : device_buffer::const_ptr(); }
	std::vector<device_buffer::const_ptr> cvec(const void * const * p, int n)
	{
		std::vector<device_buffer::const_ptr> v;
		for (int i = 0; i < n; ++i)
			v.push_back(cbuf(p[i]));
		return v;
	}
	std::vector<device_buffer::ptr> vec(void * const * p, int n)
	{
		std::vector<device_buffer::ptr> v;
		for (int i = 0; i < n; ++i)
			v.push_back(buf(p[i]));
		return v;
	}
}

#define NNFH_API extern "C" __attribute__((visibility("default")))
#define NNFH_TRY try {
#define NNFH_CATCH } catch (const std::exception& e) { g_error = e.what(); return -1; } return 0;

NNFH_API const char * nnfh_last_error() { return g_error.c_str(); }

// params: negative_slope | scale, steepness | alpha | epsilon | scale (loss) | top_n, by layer type; pool = {win_w, win_h, stride_w, stride_h, round_up_w, round_up_h, is_min}
NNFH_API void * nnfh_create(const char * type_name, int updater, const float * params, const int * pool, unsigned int feature_maps, unsigned int w, unsigned int h,
	int input_count, int with_backward)
{
	try
	{
		std::unique_ptr<handle> hd(new handle());
		hd->schema.reset(new layer());
		layer& l = *hd->schema;
		l.type_name = type_name;
		if (l.type_name == "ReLU") l.negative_slope = params[0];
		if (l.type_name == "TanH") { l.scale = params[0]; l.steepness = params[1]; }
		if (l.type_name == "Add") l.alpha = params[0];
		if (l.type_name == "NegativeLogLikelihood" || l.type_name == "CrossEntropy") l.scale = params[0];
		if (l.type_name == "Accuracy") l.top_n = (unsigned int)params[0];
		if (l.type_name == "BatchNorm") l.epsilon = params[0];
		if (l.type_name == "AverageSubsampling")
		{
			l.subsampling_sizes = {(unsigned int)pool[0], (unsigned int)pool[1]};
			l.alpha = params[0] != 0.0F ? params[0] : 1.0F; // the plain backend's default effective alpha for spatial windows
		}
		if (l.type_name == "MaxSubsampling")
		{
			l.subsampling_sizes = {(unsigned int)pool[0], (unsigned int)pool[1]};
			l.strides = {(unsigned int)pool[2], (unsigned int)pool[3]};
			l.round_ups = {pool[4] != 0, pool[5] != 0};
			l.is_min = pool[6] != 0;
		}
		layer_configuration_specific in;
		in.feature_map_count = feature_maps;
		in.dimension_sizes = {w, h};
		std::vector<layer_configuration_specific> ins(input_count, in);
		const layer_configuration_specific out = get_output_layer_configuration_specific(l, ins);
		if (updater)
		{
			std::set<layer_action> actions;
			actions.insert(layer_action(layer_action::forward));
			if (with_backward)
				actions.insert(l.type_name == "BatchNorm" ? layer_action(layer_action::backward_data_and_weights) : layer_action(layer_action::backward_data, 0));
			hd->updater = layer_factory_b200::get_singleton().create_updater(hd->schema, ins, out, actions);
		}
		else
			hd->tester = layer_factory_b200::get_singleton().create_tester(hd->schema, ins, out);
		return hd.release();
	}
	catch (const std::exception& e)
	{
		g_error = e.what();
		return nullptr;
	}
}

NNFH_API void nnfh_destroy(void * h) { delete static_cast<handle *>(h); }

NNFH_API int nnfh_tester_forward(void * h, void * stream, void * out, const void * const * data, int n_data, const void * const * inputs, int n_inputs, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->tester->enqueue_forward_propagation((cudaStream_t)stream, buf(out), {}, cvec(data, n_data), {}, cvec(inputs, n_inputs), {},
		device_buffer::ptr(), device_buffer::ptr(), entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_tester_can_write(void * h) { return static_cast<handle *>(h)->tester->get_input_index_layer_can_write(); }

NNFH_API long long nnfh_updater_query(void * h, int what, int action)
{
	layer_updater_b200& u = *static_cast<handle *>(h)->updater;
	const layer_action a((layer_action::action_type)action, action == layer_action::backward_data ? 0 : -1);
	switch (what)
	{
	case 0: return (long long)u.get_temporary_working_fixed_buffer_size(a).first;
	case 1: return (long long)u.get_temporary_fixed_buffer_size();
	case 2: return (long long)u.get_temporary_per_entry_buffer_size();
	case 3: return u.get_input_index_layer_can_write(a);
	case 4: return u.is_backward_data_dependent_on_input_buffer(0, 0);
	case 5: return u.is_backward_data_dependent_on_output_buffer(0);
	default: return -1;
	}
}

NNFH_API int nnfh_updater_forward(void * h, void * stream, void * out, const void * const * data, int n_data, const void * const * inputs, int n_inputs,
	void * working_fixed, size_t working_fixed_bytes, void * temp_fixed, void * temp_per_entry, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_forward_propagation((cudaStream_t)stream, buf(out), {}, cvec(data, n_data), {}, cvec(inputs, n_inputs), {},
		buf(working_fixed, working_fixed_bytes), device_buffer::ptr(), buf(temp_fixed), buf(temp_per_entry), entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_updater_backward_data(void * h, void * stream, void * in_err, const void * out_err, const void * const * data, int n_data,
	const void * in_neurons, const void * out_neurons, const void * temp_fixed, const void * temp_per_entry, int add_update_to_destination, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_data_propagation((cudaStream_t)stream, 0, buf(in_err), cbuf(out_err), {}, cvec(data, n_data), {},
		std::vector<device_buffer::const_ptr>(1, cbuf(in_neurons)), cbuf(out_neurons), {}, device_buffer::ptr(), device_buffer::ptr(),
		cbuf(temp_fixed), cbuf(temp_per_entry), add_update_to_destination != 0, entry_count);
	NNFH_CATCH
}

// the same for layers with several inputs (the loss layers): every input's neurons are handed over
NNFH_API int nnfh_updater_backward_data_inputs(void * h, void * stream, void * in_err, const void * out_err, const void * const * in_neurons, int n_in_neurons,
	const void * out_neurons, int add_update_to_destination, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_data_propagation((cudaStream_t)stream, 0, buf(in_err), cbuf(out_err), {}, {}, {},
		cvec(in_neurons, n_in_neurons), cbuf(out_neurons), {}, device_buffer::ptr(), device_buffer::ptr(),
		device_buffer::const_ptr(), device_buffer::const_ptr(), add_update_to_destination != 0, entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_updater_backward_weights(void * h, void * stream, void * const * gradient, int n_gradient, const void * in_neurons, const void * out_err,
	void * working_fixed, size_t working_fixed_bytes, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_weights_propagation((cudaStream_t)stream, {}, vec(gradient, n_gradient), {},
		std::vector<device_buffer::const_ptr>(1, cbuf(in_neurons)), cbuf(out_err), {}, buf(working_fixed, working_fixed_bytes), device_buffer::ptr(),
		device_buffer::const_ptr(), device_buffer::const_ptr(), entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_updater_backward_data_and_weights(void * h, void * stream, void * in_err, const void * out_err, void * const * gradient, int n_gradient,
	const void * const * data, int n_data, const void * in_neurons, void * working_fixed, size_t working_fixed_bytes, const void * temp_fixed,
	int add_update_to_destination, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_data_and_weights_propagation((cudaStream_t)stream, std::vector<device_buffer::ptr>(1, buf(in_err)), cbuf(out_err), {},
		vec(gradient, n_gradient), cvec(data, n_data), {}, std::vector<device_buffer::const_ptr>(1, cbuf(in_neurons)), device_buffer::const_ptr(), {},
		buf(working_fixed, working_fixed_bytes), device_buffer::ptr(), cbuf(temp_fixed), device_buffer::const_ptr(), add_update_to_destination != 0, entry_count);
	NNFH_CATCH
}

// ---- the same members in their general form: lists of inputs, outputs and chunks, every query --------------
// Used for the objects of fused groups (nnfh_net_*), whose heads take several inputs and may write two outputs.
NNFH_API int nnfh_forward(void * h, void * stream, void * const * outs, int n_outs, const void * const * data, int n_data, const void * const * inputs, int n_inputs,
	void * working_fixed, size_t working_fixed_bytes, void * temp_fixed, void * temp_per_entry, unsigned int entry_count)
{
	NNFH_TRY
	handle& hd = *static_cast<handle *>(h);
	if (hd.tester)
		hd.tester->enqueue_forward_propagation((cudaStream_t)stream, vec(outs, n_outs), {}, cvec(data, n_data), {}, cvec(inputs, n_inputs), {},
			buf(working_fixed, working_fixed_bytes), device_buffer::ptr(), entry_count);
	else
		hd.updater->enqueue_forward_propagation((cudaStream_t)stream, vec(outs, n_outs), {}, cvec(data, n_data), {}, cvec(inputs, n_inputs), {},
			buf(working_fixed, working_fixed_bytes), device_buffer::ptr(), buf(temp_fixed), buf(temp_per_entry), entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_backward_data(void * h, void * stream, unsigned int input_index, void * in_err, const void * out_err, const void * const * data, int n_data,
	const void * const * in_neurons, int n_in_neurons, const void * out_neurons, const void * temp_fixed, const void * temp_per_entry,
	int add_update_to_destination, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_data_propagation((cudaStream_t)stream, input_index, buf(in_err), cbuf(out_err), {}, cvec(data, n_data), {},
		cvec(in_neurons, n_in_neurons), cbuf(out_neurons), {}, device_buffer::ptr(), device_buffer::ptr(), cbuf(temp_fixed), cbuf(temp_per_entry),
		add_update_to_destination != 0, entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_backward_weights(void * h, void * stream, void * const * gradient, int n_gradient, const void * const * in_neurons, int n_in_neurons,
	const void * out_err, void * working_fixed, size_t working_fixed_bytes, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_weights_propagation((cudaStream_t)stream, {}, vec(gradient, n_gradient), {},
		cvec(in_neurons, n_in_neurons), cbuf(out_err), {}, buf(working_fixed, working_fixed_bytes), device_buffer::ptr(),
		device_buffer::const_ptr(), device_buffer::const_ptr(), entry_count);
	NNFH_CATCH
}

NNFH_API int nnfh_backward_data_and_weights(void * h, void * stream, void * const * in_errs, int n_in_errs, const void * out_err, void * const * gradient, int n_gradient,
	const void * const * data, int n_data, const void * const * in_neurons, int n_in_neurons, const void * out_neurons, void * working_fixed, size_t working_fixed_bytes,
	const void * temp_fixed, int add_update_to_destination, unsigned int entry_count)
{
	NNFH_TRY
	static_cast<handle *>(h)->updater->enqueue_backward_data_and_weights_propagation((cudaStream_t)stream, vec(in_errs, n_in_errs), cbuf(out_err), {},
		vec(gradient, n_gradient), cvec(data, n_data), {}, cvec(in_neurons, n_in_neurons), cbuf(out_neurons), {},
		buf(working_fixed, working_fixed_bytes), device_buffer::ptr(), cbuf(temp_fixed), device_buffer::const_ptr(), add_update_to_destination != 0, entry_count);
	NNFH_CATCH
}

// what: 0 temporary_working_fixed size, 1 temporary_fixed size, 2 temporary_per_entry size, 3 input index the layer can write,
// 4-7 backward_data depends on input buffer b / output buffer / temporary fixed / temporary per entry (a = action input index),
// 8-11 the same for backward_data_and_weights, 12-14 backward_weights on input buffer b / temporary fixed / temporary per entry,
// 15 output count, 16 temporary_working_per_entry size, 17 persistent working buffers, 18 inputs read through a texture
NNFH_API long long nnfh_query(void * h, int what, int action_type, int backprop_index, unsigned int a, unsigned int b)
{
	handle& hd = *static_cast<handle *>(h);
	const layer_action act((layer_action::action_type)action_type, backprop_index);
	try
	{
		if (hd.tester)
		{
			layer_tester_b200& t = *hd.tester;
			switch (what)
			{
			case 0: return (long long)t.get_temporary_working_fixed_buffer_size().first;
			case 3: return t.get_input_index_layer_can_write();
			case 15: return t.get_output_count();
			case 16: return (long long)t.get_temporary_working_per_entry_buffer_size();
			case 17: return (long long)t.get_persistent_working_data().size();
			case 18: return (long long)t.get_linear_addressing_through_texture_per_entry().size();
			default: return -1;
			}
		}
		layer_updater_b200& u = *hd.updater;
		switch (what)
		{
		case 0: return (long long)u.get_temporary_working_fixed_buffer_size(act).first;
		case 1: return (long long)u.get_temporary_fixed_buffer_size();
		case 2: return (long long)u.get_temporary_per_entry_buffer_size();
		case 3: return u.get_input_index_layer_can_write(act);
		case 4: return u.is_backward_data_dependent_on_input_buffer(a, b);
		case 5: return u.is_backward_data_dependent_on_output_buffer(a);
		case 6: return u.is_backward_data_dependent_on_temporary_fixed_buffer(a);
		case 7: return u.is_backward_data_dependent_on_temporary_per_entry_buffer(a);
		case 8: return u.is_backward_data_and_weights_dependent_on_input_buffer(b);
		case 9: return u.is_backward_data_and_weights_dependent_on_output_buffer();
		case 10: return u.is_backward_data_and_weights_dependent_on_temporary_fixed_buffer();
		case 11: return u.is_backward_data_and_weights_dependent_on_temporary_per_entry_buffer();
		case 12: return u.is_backward_weights_dependent_on_input_buffer(b);
		case 13: return u.is_backward_weights_dependent_on_temporary_fixed_buffer();
		case 14: return u.is_backward_weights_dependent_on_temporary_per_entry_buffer();
		case 15: return u.get_output_count();
		case 16: return (long long)u.get_temporary_working_per_entry_buffer_size(act);
		case 17: return (long long)u.get_persistent_working_data().size();
		case 18: return (long long)u.get_linear_addressing_through_texture_per_entry().size();
		default: return -1;
		}
	}
	catch (const std::exception& e)
	{
		g_error = e.what();
		return -2;
	}
}

// Weights to the device through the object's get_data; the device pointers land in out_device (one per chunk) and stay
// valid while the handle lives. nnfh_get_data_from_device copies them back through get_data_from_device (updaters).
NNFH_API int nnfh_get_data(void * h, const float * const * parts, const long long * elem_counts, int n_parts, void ** out_device)
{
	NNFH_TRY
	handle& hd = *static_cast<handle *>(h);
	layer_data::ptr host(new layer_data());
	for (int i = 0; i < n_parts; ++i)
		host->push_back(std::vector<float>(parts[i], parts[i] + elem_counts[i]));
	hd.uploaded.clear();
	hd.uploaded_const.clear();
	if (hd.tester)
	{
		hd.uploaded_const = hd.tester->get_data(host);
		for (int i = 0; i < n_parts; ++i)
			out_device[i] = const_cast<void *>(static_cast<const void *>(*hd.uploaded_const[i]));
	}
	else
	{
		hd.uploaded = hd.updater->get_data(host);
		for (int i = 0; i < n_parts; ++i)
			out_device[i] = static_cast<void *>(*hd.uploaded[i]);
	}
	NNFH_CATCH
}

NNFH_API int nnfh_get_data_from_device(void * h, float * const * parts, const long long * elem_counts, int n_parts)
{
	NNFH_TRY
	handle& hd = *static_cast<handle *>(h);
	if (!hd.updater || (int)hd.uploaded.size() != n_parts)
		throw neural_network_exception("nnfh_get_data_from_device: call nnfh_get_data on an updater first");
	layer_data::ptr host(new layer_data());
	for (int i = 0; i < n_parts; ++i)
		host->push_back(std::vector<float>((size_t)elem_counts[i]));
	hd.updater->get_data_from_device(hd.uploaded, host);
	for (int i = 0; i < n_parts; ++i)
		std::memcpy(parts[i], (*host)[i].data(), (size_t)elem_counts[i] * sizeof(float));
	NNFH_CATCH
}

// the fields of running_configuration_b200 for the current device: device_id, compute capability major and minor,
// multiprocessor_count, max_threads_per_multiprocessor, smem_per_block, smem_per_multiprocessor, l2_cache_size,
// max_registers_per_multiprocessor, device_pos, device_count
NNFH_API int nnfh_running_configuration(long long * out11)
{
	NNFH_TRY
	const running_configuration_b200::const_ptr rc = running_configuration_b200::get_current();
	const long long v[11] = {rc->device_id, rc->compute_capability_major, rc->compute_capability_minor, rc->multiprocessor_count,
		rc->max_threads_per_multiprocessor, (long long)rc->smem_per_block, (long long)rc->smem_per_multiprocessor, rc->l2_cache_size,
		rc->max_registers_per_multiprocessor, rc->device_pos, rc->device_count};
	std::memcpy(out11, v, sizeof(v));
	NNFH_CATCH
}

// One layer's chunks: sizes in elements; prev_upd / prev_upd2 / update_accum may be null
NNFH_API int nnfh_apply_gradient(void * stream, int n_parts, void * const * data, void * const * gradient, void * const * prev_upd, void * const * prev_upd2,
	void * const * update_accum, const float * learning_rates, const long long * elem_counts, const int * weight_decay_parts, int n_weight_decay_parts,
	float gradient_normalizer, float weight_decay, int momentum_type, float momentum_val, float momentum_val2, unsigned int iteration_id)
{
	NNFH_TRY
	auto sized = [&](void * const * p) {
		std::vector<device_buffer::ptr> v;
		for (int i = 0; p && i < n_parts; ++i)
			v.push_back(device_buffer::ptr(new device_buffer(p[i], size_t(elem_counts[i]) * sizeof(float))));
		return std::vector<std::vector<device_buffer::ptr>>(1, v);
	};
	std::vector<std::vector<device_buffer::ptr>> accum;
	if (update_accum)
		accum = sized(update_accum);
	enqueue_apply_gradient((cudaStream_t)stream, sized(data), sized(gradient), sized(prev_upd), sized(prev_upd2),
		std::vector<std::vector<float>>(1, std::vector<float>(learning_rates, learning_rates + n_parts)), accum,
		std::vector<std::set<unsigned int>>(1, std::set<unsigned int>(weight_decay_parts, weight_decay_parts + n_weight_decay_parts)),
		gradient_normalizer, weight_decay, training_momentum((training_momentum::momentum_type)momentum_type, momentum_val, momentum_val2), iteration_id);
	NNFH_CATCH
}
