// Host-side layer objects over the nnf_b200 C ABI, shaped like nnForge's CUDA backend objects:
// a `layer_tester_b200` answers and enqueues what nnforge::cuda::layer_tester_cuda does
// (nnforge/cuda/layer_tester_cuda.h:47-72), a `layer_updater_b200` what layer_updater_cuda does
// (nnforge/cuda/layer_updater_cuda.h:50-169), and both are created through string-keyed factories by
// the reference's layer type names ("BatchNorm", "ReLU", "PReLU", "ELU", "TanH", "Sigmoid", "Softmax",
// "Add", "MaxSubsampling", and their neighbours "AverageSubsampling", "NegativeLogLikelihood", "CrossEntropy", "Accuracy";
// nnforge/cuda/layer_testing_schema_factory.cpp:36-44). Method names, argument
// order and meaning, buffer-plan queries and the error convention (exceptions derived from
// std::runtime_error thrown on the calling host thread) are the reference's, so an nnForge scheduler
// can drive these objects the way it drives its own; the arithmetic behind them is libnnf_b200.
//
// The small value types below (layer description, shape, action, buffer, weights, running configuration)
// stand in for nnForge's layer / layer_configuration_specific / layer_action / cuda_linear_buffer_device /
// layer_data / cuda_running_configuration, whose headers cannot be compiled without Boost and protobuf.
//
// Two things go beyond the reference's interface, both for fused groups (nnf_fusion.h): the overload of
// enqueue_forward_propagation that takes a LIST of output buffers (a fused head may write two layer
// outputs in one pass), and layer_factory_b200::create_testers / create_updaters, which turn a planned
// group into one head object plus no-op follower objects.
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>
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
		std::string instance_name;                  // layer::instance_name
		float epsilon = 2.0e-5F;                    // BatchNorm (default_batch_normalization_epsilon, nnforge/batch_norm_layer.cpp:28)
		float negative_slope = 0.0F;                // ReLU
		float scale = 1.0F, steepness = 1.0F;       // TanH; scale also NegativeLogLikelihood, CrossEntropy
		float alpha = 1.0F;                         // Add; AverageSubsampling: the effective alpha
		unsigned int top_n = 1;                     // Accuracy
		std::vector<unsigned int> subsampling_sizes; // MaxSubsampling, AverageSubsampling
		std::vector<unsigned int> strides;
		std::vector<bool> round_ups;
		unsigned int feature_map_subsampling_size = 1, entry_subsampling_size = 1;
		bool is_min = false, tiling = false;
	};

	// nnforge/layer_data.h, layer_data_custom.h: the weight chunks of one layer on the host
	struct layer_data : public std::vector<std::vector<float>>
	{
		typedef std::shared_ptr<layer_data> ptr;
		typedef std::shared_ptr<const layer_data> const_ptr;
	};
	struct layer_data_custom : public std::vector<std::vector<int>>
	{
		typedef std::shared_ptr<layer_data_custom> ptr;
		typedef std::shared_ptr<const layer_data_custom> const_ptr;
	};

	// nnforge/buffer_lifetime.h:23-69: which of a layer's buffers a scheduler is planning
	class buffer_lifetime
	{
	public:
		enum buffer_lifetime_type { action_output_buffer = 0, working_buffer = 1, temporary_buffer = 2 };
		buffer_lifetime(buffer_lifetime_type blt = action_output_buffer) : blt(blt) {}
		buffer_lifetime_type get_buffer_lifetime_type() const { return blt; }
		std::string str() const { return blt == action_output_buffer ? "action_output" : blt == working_buffer ? "working" : blt == temporary_buffer ? "temporary" : ""; }
		bool operator<(const buffer_lifetime& o) const { return (unsigned int)blt < (unsigned int)o.blt; }
	private:
		buffer_lifetime_type blt;
	};

	// Device memory (nnforge/cuda/cuda_linear_buffer_device.cpp:28-73). The two-argument form is a
	// non-owning view of memory the scheduler owns (a layer never frees or keeps one); the one-argument
	// form allocates, like the reference's constructor, and is used at set-up time only (weights,
	// persistent working data) - never while enqueueing.
	class device_buffer
	{
	public:
		typedef std::shared_ptr<device_buffer> ptr;
		typedef std::shared_ptr<const device_buffer> const_ptr;
		device_buffer(void * p, size_t bytes) : p(p), bytes(bytes) {}
		explicit device_buffer(size_t bytes);
		~device_buffer();
		device_buffer(const device_buffer&) = delete;
		device_buffer& operator=(const device_buffer&) = delete;
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
		bool owned = false;
	};

	// Where the devices that share a batch leave the addresses of the buffers their layers exchange
	// statistics through (the mailboxes of the batch-sharded batch norm). nnForge runs its GPUs from one
	// process (nnforge/cuda/cuda_multi_running_configuration.h), so one directory object is shared by the
	// running configurations of all devices; with one process per GPU each process publishes, BEFORE it
	// creates its layer objects, its own buffer (one that the other processes can map, zero-filled) under
	// its own position and the addresses its mappings of the other processes' buffers gave it under
	// theirs: a layer that finds its own position filled uses that buffer instead of allocating one.
	// Thread-safe.
	class peer_directory
	{
	public:
		typedef std::shared_ptr<peer_directory> ptr;
		void publish(const std::string& key, int device_pos, void * address);
		// the address published for one position, or null
		void * find(const std::string& key, int device_pos) const;
		// addresses by device position; throws neural_network_exception while any position is missing
		std::vector<void *> lookup(const std::string& key, int device_count) const;
	private:
		mutable std::mutex m;
		std::map<std::string, std::map<int, void *>> entries;
	};

	// The public fields of cuda_running_configuration that this path reads (nnforge/cuda/cuda_running_configuration.h:126-153),
	// filled from the device's attributes. device_pos / device_count / peers describe the set of devices
	// that share a batch (cuda_multi_running_configuration); a single device has position 0 of 1.
	class running_configuration_b200
	{
	public:
		typedef std::shared_ptr<running_configuration_b200> ptr;
		typedef std::shared_ptr<const running_configuration_b200> const_ptr;

		explicit running_configuration_b200(int device_id, int device_pos = 0, int device_count = 1, peer_directory::ptr peers = peer_directory::ptr());

		// the configuration of the device that is current on the calling thread (cached per device)
		static const_ptr get_current();

		int get_compute_capability() const { return compute_capability_major * 100 + compute_capability_minor; }
		void set_device() const;

		int device_id;
		int device_pos;
		int device_count;
		peer_directory::ptr peers;

		int compute_capability_major = 0;
		int compute_capability_minor = 0;
		int multiprocessor_count = 0;
		int max_threads_per_multiprocessor = 0;
		size_t smem_per_block = 0;            // the opt-in maximum a kernel of this library may ask for
		size_t smem_per_multiprocessor = 0;
		int l2_cache_size = 0;
		int max_registers_per_multiprocessor = 0;
	};

	class layer_tester_b200
	{
	public:
		typedef std::shared_ptr<layer_tester_b200> ptr;
		virtual ~layer_tester_b200() = default;

		void configure(
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific,
			layer::const_ptr layer_schema,
			running_configuration_b200::const_ptr cuda_config = running_configuration_b200::const_ptr());

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

		// The same call with one buffer per layer output the object writes (get_output_count() of them). Objects with
		// one output forward to the member above; the heads of fused groups that write two layer outputs in one pass
		// (the ReLU output and the pooled tensor; the probabilities and the loss) implement this form only.
		virtual void enqueue_forward_propagation(
			cudaStream_t stream_id,
			const std::vector<device_buffer::ptr>& output_buffers,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::const_ptr>& data,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_buffers,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			unsigned int entry_count);
		virtual unsigned int get_output_count() const { return 1; }

		// Weights to the device, one buffer per chunk (nnforge/cuda/layer_tester_cuda.cpp: get_data, set_get_data_custom)
		virtual std::vector<device_buffer::const_ptr> get_data(layer_data::const_ptr host_data) const;
		virtual std::vector<device_buffer::const_ptr> set_get_data_custom(layer_data_custom::const_ptr host_data);
		virtual std::vector<device_buffer::const_ptr> get_persistent_working_data() const { return std::vector<device_buffer::const_ptr>(); }

		virtual int get_input_index_layer_can_write() const { return -1; }
		virtual std::pair<size_t, bool> get_temporary_working_fixed_buffer_size() const { return std::make_pair(size_t(0), false); }
		virtual size_t get_temporary_working_per_entry_buffer_size() const { return 0; }
		// no layer of this path reads its input through a texture
		virtual std::vector<unsigned int> get_linear_addressing_through_texture_per_entry() const { return std::vector<unsigned int>(); }

	protected:
		virtual void tester_configured() {}
		virtual void notify_data_custom(layer_data_custom::const_ptr host_data_custom) {}
		layer::const_ptr layer_schema;
		running_configuration_b200::const_ptr cuda_config;
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
			running_configuration_b200::const_ptr cuda_config,
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

		// The same call with one buffer per layer output the object writes; see layer_tester_b200.
		virtual void enqueue_forward_propagation(
			cudaStream_t stream_id,
			const std::vector<device_buffer::ptr>& output_buffers,
			const std::vector<device_buffer::const_ptr>& schema_data,
			const std::vector<device_buffer::const_ptr>& data,
			const std::vector<device_buffer::const_ptr>& data_custom,
			const std::vector<device_buffer::const_ptr>& input_buffers,
			const std::vector<device_buffer::const_ptr>& persistent_working_data,
			device_buffer::ptr temporary_working_fixed_buffer,
			device_buffer::ptr temporary_working_per_entry_buffer,
			device_buffer::ptr temporary_fixed_buffer,
			device_buffer::ptr temporary_per_entry_buffer,
			unsigned int entry_count);
		virtual unsigned int get_output_count() const { return 1; }

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

		// Weights to the device and back, one buffer per chunk (nnforge/cuda/layer_updater_cuda.cpp:67-107)
		virtual std::vector<device_buffer::ptr> get_data(layer_data::const_ptr host_data) const;
		virtual std::vector<device_buffer::const_ptr> set_get_data_custom(layer_data_custom::const_ptr host_data);
		// buffers the object itself owns for as long as it lives (default: none)
		virtual std::vector<device_buffer::const_ptr> get_persistent_working_data() const { return std::vector<device_buffer::const_ptr>(); }
		void get_data_from_device(const std::vector<device_buffer::ptr>& device_data, layer_data::ptr host_data) const;
		// no layer of this path reads its input through a texture
		virtual std::vector<unsigned int> get_linear_addressing_through_texture_per_entry() const { return std::vector<unsigned int>(); }

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
		virtual bool is_backward_data_and_weights_dependent_on_temporary_fixed_buffer() const { return get_temporary_fixed_buffer_size() != 0; }
		virtual bool is_backward_data_and_weights_dependent_on_temporary_per_entry_buffer() const { return get_temporary_per_entry_buffer_size() != 0; }
		virtual bool is_backward_weights_dependent_on_input_buffer(unsigned int data_input_index) const { return true; }
		virtual bool is_backward_weights_dependent_on_temporary_fixed_buffer() const { return get_temporary_fixed_buffer_size() != 0; }
		virtual bool is_backward_weights_dependent_on_temporary_per_entry_buffer() const { return get_temporary_per_entry_buffer_size() != 0; }

	protected:
		virtual void updater_configured() {}
		virtual void notify_data_custom(layer_data_custom::const_ptr host_data_custom) {}
		layer::const_ptr layer_schema;
		running_configuration_b200::const_ptr cuda_config;
		std::vector<layer_configuration_specific> input_configuration_specific_list;
		layer_configuration_specific output_configuration_specific;
		unsigned int output_elem_count_per_entry = 0;
		unsigned int output_elem_count_per_feature_map = 0;
		std::set<layer_action> actions;
	};

	struct schema_node;
	struct fused_group;

	// How a scheduler feeds the head object of a fused group. Node indices refer to the schema list that was
	// given to plan_fusion. The head stands for the whole group: it runs where the group's first member would
	// run, reads the group's inputs, carries the followers' parameters and writes the outputs the group
	// materialises; the other members' objects do nothing.
	struct fused_io
	{
		// element k of the head's input_buffers (forward) / input_neurons_buffers, and of input_errors_buffers
		// in backward_data_and_weights: input number .second of node .first
		std::vector<std::pair<int, unsigned int>> input_sources;
		// the head's data (and gradient) list: the chunks of these nodes, concatenated in this order
		std::vector<int> data_sources;
		// the nodes whose output buffers the head writes, in the order of its output buffer list. One element:
		// the plain enqueue_forward_propagation; two: the overload taking a list. In backward, the head's
		// output_errors_buffer is the error of the LAST of them and output_neurons_buffer the FIRST.
		std::vector<int> output_sources;
	};

	struct fused_testers
	{
		std::vector<layer_tester_b200::ptr> objects; // one per member, in member order; objects[0] is the head
		fused_io io;
	};

	struct fused_updaters
	{
		std::vector<layer_updater_b200::ptr> objects; // one per member, in member order; objects[0] is the head
		fused_io io;
	};

	// String-keyed prototypes, like layer_testing_schema_factory / layer_updater_schema_factory
	// (nnforge/cuda/layer_testing_schema.cpp:25-51: the schema's create_tester configures the new object with the
	// shapes and the cuda_running_configuration). cuda_config may be empty: the current device's is then used.
	class layer_factory_b200
	{
	public:
		static layer_factory_b200& get_singleton();

		// throws neural_network_exception for a type name that is not registered
		layer_tester_b200::ptr create_tester(
			layer::const_ptr layer_schema,
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific,
			running_configuration_b200::const_ptr cuda_config = running_configuration_b200::const_ptr()) const;

		layer_updater_b200::ptr create_updater(
			layer::const_ptr layer_schema,
			const std::vector<layer_configuration_specific>& input_configuration_specific_list,
			const layer_configuration_specific& output_configuration_specific,
			const std::set<layer_action>& actions,
			running_configuration_b200::const_ptr cuda_config = running_configuration_b200::const_ptr()) const;

		// The objects of one planned group (nnf_fusion.h). For a fused kind: a head that calls the group's fused
		// entry point of the C ABI plus one follower per remaining member, whose enqueue_* members do nothing and
		// whose get_input_index_layer_can_write answers 0 so that a per-layer buffer plan keeps them on the
		// head's buffer. For fused_single_layer: the one object create_tester / create_updater would return.
		// output_configurations maps a layer instance name to its output shape: every node of the list, and the
		// data layers the list reads from.
		fused_testers create_testers(
			const fused_group& group,
			const std::vector<schema_node>& nodes,
			const std::map<std::string, layer_configuration_specific>& output_configurations,
			running_configuration_b200::const_ptr cuda_config = running_configuration_b200::const_ptr()) const;

		// actions: per member, what that layer would be configured with on its own
		fused_updaters create_updaters(
			const fused_group& group,
			const std::vector<schema_node>& nodes,
			const std::map<std::string, layer_configuration_specific>& output_configurations,
			const std::vector<std::set<layer_action>>& actions,
			running_configuration_b200::const_ptr cuda_config = running_configuration_b200::const_ptr()) const;

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
