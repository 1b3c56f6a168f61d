// Host-side layer objects over the nnf_b200 C ABI, shaped like nnForge's CUDA backend objects:
// a `layer_tester_b200` answers and enqueues what nnforge::cuda::layer_tester_cuda does
// (nnforge/cuda/layer_tester_cuda.h:47-72), a `layer_updater_b200` what layer_updater_cuda does
// (nnforge/cuda/layer_updater_cuda.h:50-169), and both are created through string-keyed factories by
// the reference's layer type names ("BatchNorm", "ReLU", "PReLU", "ELU", "TanH", "Sigmoid", "Softmax",
// "Add", "MaxSubsampling"; nnforge/cuda/layer_testing_schema_factory.cpp:36-44). Method names, argument
// order and meaning, buffer-plan queries and the error convention (exceptions derived from
// std::runtime_error thrown on the calling host thread) are the reference's, so an nnForge scheduler
// can drive these objects the way it drives its own; the arithmetic behind them is libnnf_b200.
//
// The small value types below (layer description, shape, action, buffer) stand in for nnForge's
// layer / layer_configuration_specific / layer_action / cuda_linear_buffer_device, whose headers
// cannot be compiled without Boost and protobuf.
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace nnf_b200
{
	class neural_network_exception : public std::runtime_error
	{
	public:
		explicit neural_network_exception(const std::string& message) : std::runtime_error(message) {}
	};

	// nnforge/layer_configuration_specific.h:27-64 (dimension_sizes[0] is the fastest dimension, x)
	struct layer_configuration_specific
	{
		unsigned int feature_map_count = 0;
		std::vector<unsigned int> dimension_sizes;

		unsigned int get_neuron_count_per_feature_map() const
		{
			unsigned int r = 1;
			for (unsigned int d : dimension_sizes)
				r *= d;
			return r;
		}
		unsigned int get_neuron_count() const { return feature_map_count * get_neuron_count_per_feature_map(); }
	};

	// nnforge/layer_action.h:24-90
	struct layer_action
	{
		enum action_type { forward = 0, backward_data = 1, backward_weights = 2, backward_data_and_weights = 3, update_weights = 4 };
		action_type at;
		int backprop_index;
		layer_action(action_type at = forward, int backprop_index = -1) : at(at), backprop_index(backprop_index) {}
		action_type get_action_type() const { return at; }
		bool operator<(const layer_action& o) const { return at != o.at ? at < o.at : backprop_index < o.backprop_index; }
	};

	// The parameters the nine layer classes carry (nnforge/batch_norm_layer.h, rectified_linear_layer.h,
	// hyperbolic_tangent_layer.h, add_layer.h, max_subsampling_layer.h ...), by the reference's field names.
	struct layer
	{
		typedef std::shared_ptr<const layer> const_ptr;
		std::string type_name;                      // layer::get_type_name()
		float epsilon = 2.0e-5F;                    // BatchNorm (default_batch_normalization_epsilon, nnforge/batch_norm_layer.cpp:28)
		float negative_slope = 0.0F;                // ReLU
		float scale = 1.0F, steepness = 1.0F;       // TanH; scale also NegativeLogLikelihood
		float alpha = 1.0F;                         // Add; AverageSubsampling: the effective alpha
		unsigned int top_n = 1;                     // Accuracy
		std::vector<unsigned int> subsampling_sizes; // MaxSubsampling, AverageSubsampling
		std::vector<unsigned int> strides;
		std::vector<bool> round_ups;
		unsigned int feature_map_subsampling_size = 1, entry_subsampling_size = 1;
		bool is_min = false, tiling = false;
	};

	// Device memory handed over by the scheduler (nnforge/cuda/cuda_linear_buffer_device.h). Non-owning
	// views are enough here: the scheduler owns every buffer, a layer never frees or keeps one.
	class device_buffer
	{
	public:
		typedef std::shared_ptr<device_buffer> ptr;
		typedef std::shared_ptr<const device_buffer> const_ptr;
		device_buffer(void * p, size_t bytes) : p(p), bytes(bytes) {}
		operator float *() { return static_cast<float *>(p); }
		operator const float *() const { return static_cast<const float *>(p); }
		operator void *() { return p; }
		operator const void *() const { return p; }
		operator unsigned int *() { return static_cast<unsigned int *>(p); }
		operator const unsigned int *() const { return static_cast<const unsigned int *>(p); }
		size_t get_size() const { return bytes; }
	private:
		void * p;
		size_t bytes;
	};

	class layer_tester_b200
	{
	public:
		typedef std::shared_ptr<layer_tester_b200> ptr;
		virtual ~layer_tester_b200() = default;

		void configure(
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific,
			layer::const_ptr layer_schema);

		virtual void enqueue_forward_propagation(
			cudaStream_t stream_id,
			device_buffer::ptr output_buffer,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::const_ptr>& data,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_buffers,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			unsigned int entry_count) = 0;

		virtual int get_input_index_layer_can_write() const { return -1; }
		virtual std::pair<size_t, bool> get_temporary_working_fixed_buffer_size() const { return std::make_pair(size_t(0), false); }
		virtual size_t get_temporary_working_per_entry_buffer_size() const { return 0; }

	protected:
		virtual void tester_configured() {}
		layer::const_ptr layer_schema;
		std::vector<layer_configuration_specific> input_configuration_specific_list;
		layer_configuration_specific output_configuration_specific;
		unsigned int output_elem_count_per_entry = 0;
		unsigned int output_elem_count_per_feature_map = 0;
	};

	class layer_updater_b200
	{
	public:
		typedef std::shared_ptr<layer_updater_b200> ptr;
		virtual ~layer_updater_b200() = default;

		void configure(
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific,
			layer::const_ptr layer_schema,
			const std::set<layer_action>& actions);

		virtual void enqueue_forward_propagation(
			cudaStream_t stream_id,
			device_buffer::ptr output_buffer,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::const_ptr>& data,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_buffers,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			device_buffer::ptr temporary_fixed_buffer,
			device_buffer::ptr temporary_per_entry_buffer,
			unsigned int entry_count) = 0;

		virtual void enqueue_backward_data_propagation(
			cudaStream_t stream_id,
			unsigned int input_index,
			device_buffer::ptr input_errors_buffer,
			device_buffer::const_ptr output_errors_buffer,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::const_ptr>& data,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_neurons_buffers,
			device_buffer::const_ptr output_neurons_buffer,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			device_buffer::const_ptr temporary_fixed_buffer,
			device_buffer::const_ptr temporary_per_entry_buffer,
			bool add_update_to_destination,
			unsigned int entry_count);

		virtual void enqueue_backward_weights_propagation(
			cudaStream_t stream_id,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::ptr>& gradient,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_neurons_buffers,
			device_buffer::const_ptr output_errors_buffer,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			device_buffer::const_ptr temporary_fixed_buffer,
			device_buffer::const_ptr temporary_per_entry_buffer,
			unsigned int entry_count);

		virtual void enqueue_backward_data_and_weights_propagation(
			cudaStream_t stream_id,
			const std::vector<device_buffer::ptr> input_errors_buffers,
			device_buffer::const_ptr output_errors_buffer,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::ptr>& gradient,
			const std::vector<device_buffer::const_ptr>& data,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_neurons_buffers,
			device_buffer::const_ptr output_neurons_buffer,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			device_buffer::const_ptr temporary_fixed_buffer,
			device_buffer::const_ptr temporary_per_entry_buffer,
			bool add_update_to_destination,
			unsigned int entry_count);

		// The function returns the minimum size and whether the updater would like a larger buffer
		virtual std::pair<size_t, bool> get_temporary_working_fixed_buffer_size(const layer_action& action) const { return std::make_pair(size_t(0), false); }
		virtual size_t get_temporary_working_per_entry_buffer_size(const layer_action& action) const { return 0; }
		virtual size_t get_temporary_fixed_buffer_size() const { return 0; }     // created in forward, used in backward
		virtual size_t get_temporary_per_entry_buffer_size() const { return 0; } // created in forward, used in backward
		virtual int get_input_index_layer_can_write(const layer_action& action) const { return -1; }
		virtual bool is_backward_data_dependent_on_input_buffer(unsigned int action_input_index, unsigned int data_input_index) const { return true; }
		virtual bool is_backward_data_dependent_on_output_buffer(unsigned int action_input_index) const { return true; }
		virtual bool is_backward_data_dependent_on_temporary_fixed_buffer(unsigned int action_input_index) const { return get_temporary_fixed_buffer_size() != 0; }
		virtual bool is_backward_data_dependent_on_temporary_per_entry_buffer(unsigned int action_input_index) const { return get_temporary_per_entry_buffer_size() != 0; }
		virtual bool is_backward_data_and_weights_dependent_on_input_buffer(unsigned int data_input_index) const { return true; }
		virtual bool is_backward_data_and_weights_dependent_on_output_buffer() const { return true; }
		virtual bool is_backward_weights_dependent_on_input_buffer(unsigned int data_input_index) const { return true; }

	protected:
		virtual void updater_configured() {}
		layer::const_ptr layer_schema;
		std::vector<layer_configuration_specific> input_configuration_specific_list;
		layer_configuration_specific output_configuration_specific;
		unsigned int output_elem_count_per_entry = 0;
		unsigned int output_elem_count_per_feature_map = 0;
		std::set<layer_action> actions;
	};

	// String-keyed prototypes, like layer_testing_schema_factory / layer_updater_schema_factory.
	class layer_factory_b200
	{
	public:
		static layer_factory_b200& get_singleton();

		// throws neural_network_exception for a type name that is not one of the nine
		layer_tester_b200::ptr create_tester(
			layer::const_ptr layer_schema,
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific) const;

		layer_updater_b200::ptr create_updater(
			layer::const_ptr layer_schema,
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific,
			const std::set<layer_action>& actions) const;

		std::vector<std::string> get_type_names() const;
	};

	// nnforge/training_momentum.h
	struct training_momentum
	{
		enum momentum_type { no_momentum, vanilla_momentum, nesterov_momentum, adam_momentum };
		training_momentum(momentum_type type = no_momentum, float momentum_val = 0.0F, float momentum_val2 = 0.0F)
			: type(type), momentum_val(momentum_val), momentum_val2(momentum_val2) {}
		bool is_momentum_data() const { return type != no_momentum; }
		bool is_momentum_data2() const { return type == adam_momentum; }
		momentum_type type;
		float momentum_val, momentum_val2;
	};

	// The optimiser step of backward_propagation_cuda::enqueue_apply_gradient (nnforge/cuda/backward_propagation_cuda.cpp:2008-2096)
	// for ALL weight chunks of ALL layers given, in one launch per 48 chunks instead of one launch per chunk. One element of
	// each list per layer; data[l][part] sizes give the element counts; update_accum_buffers[l] may be empty (no statistics)
	// or hold one buffer of one double per chunk. weight_decay applies to the chunks in weight_decay_part_ids[l]
	// (layer::get_weight_decay_part_id_set(): empty for BatchNorm and PReLU).
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
		unsigned int iteration_id);

	// Output shape of a layer for given inputs (max_subsampling_layer.cpp:106-137; identity for the rest).
	layer_configuration_specific get_output_layer_configuration_specific(const layer& l, const std::vector<layer_configuration_specific>& inputs);
}
