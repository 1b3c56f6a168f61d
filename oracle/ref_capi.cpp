// Flat C entry points over nnForge's own plain (CPU) backend classes, compiled together with the
// reference's unmodified sources (see oracle/build_ref.py). TEST INFRASTRUCTURE ONLY: it exists to
// pin the C restatement in oracle/nnf_oracle.c and to time the reference CPU path; nothing in the
// product library links or loads it.
//
// Every function builds the layer object, plain_buffers and configuration objects exactly the way
// nnforge/plain/forward_propagation_plain.cpp:150-186 and backward_propagation_plain.cpp:297-433
// hand them to run_forward_propagation / run_backward_*_propagation, copies caller data in, runs
// the call `reps` times, copies results out and returns the best wall time of the run call alone
// (seconds). A negative return value means the reference threw; ref_last_error() has the text.
#include "plain/batch_norm_layer_tester_plain.h"
#include "plain/rectified_linear_layer_tester_plain.h"
#include "plain/rectified_linear_layer_updater_plain.h"
#include "plain/parametric_rectified_linear_layer_tester_plain.h"
#include "plain/parametric_rectified_linear_layer_updater_plain.h"
#include "plain/exponential_linear_layer_tester_plain.h"
#include "plain/exponential_linear_layer_updater_plain.h"
#include "plain/hyperbolic_tangent_layer_tester_plain.h"
#include "plain/hyperbolic_tangent_layer_updater_plain.h"
#include "plain/sigmoid_layer_tester_plain.h"
#include "plain/sigmoid_layer_updater_plain.h"
#include "plain/softmax_layer_tester_plain.h"
#include "plain/softmax_layer_updater_plain.h"
#include "plain/negative_log_likelihood_layer_tester_plain.h"
#include "plain/negative_log_likelihood_layer_updater_plain.h"
#include "plain/cross_entropy_layer_tester_plain.h"
#include "plain/cross_entropy_layer_updater_plain.h"
#include "plain/accuracy_layer_tester_plain.h"
#include "plain/accuracy_layer_updater_plain.h"
#include "plain/average_subsampling_layer_tester_plain.h"
#include "plain/average_subsampling_layer_updater_plain.h"
#include "plain/add_layer_tester_plain.h"
#include "plain/add_layer_updater_plain.h"
#include "plain/max_subsampling_layer_tester_plain.h"
#include "plain/max_subsampling_layer_updater_plain.h"

#include "batch_norm_layer.h"
#include "rectified_linear_layer.h"
#include "parametric_rectified_linear_layer.h"
#include "exponential_linear_layer.h"
#include "hyperbolic_tangent_layer.h"
#include "sigmoid_layer.h"
#include "softmax_layer.h"
#include "negative_log_likelihood_layer.h"
#include "cross_entropy_layer.h"
#include "accuracy_layer.h"
#include "average_subsampling_layer.h"
#include "add_layer.h"
#include "max_subsampling_layer.h"
#include "stat_data_bunch_writer.h"

#include <chrono>
#include <cstring>
#include <string>

using namespace nnforge;
using namespace nnforge::plain;

namespace
{
	std::string g_last_error;

	typedef std::chrono::steady_clock clk;

	plain_buffer::ptr make_buffer(const void * src, size_t bytes)
	{
		plain_buffer::ptr b(new plain_buffer(bytes == 0 ? 4 : bytes));
		if (src && bytes)
			memcpy((void *)(*b), src, bytes);
		return b;
	}

	layer_configuration_specific make_config(unsigned int c, unsigned int h, unsigned int w)
	{
		std::vector<unsigned int> dims;
		dims.push_back(w);
		dims.push_back(h);
		return layer_configuration_specific(c, dims);
	}

	plain_running_configuration::const_ptr make_running_config(int threads)
	{
		return plain_running_configuration::const_ptr(new plain_running_configuration(threads < 1 ? 1 : threads, 16.0F));
	}

	template <class F>
	double timed(int reps, F f)
	{
		double best = 1.0e30;
		for (int r = 0; r < (reps < 1 ? 1 : reps); ++r)
		{
			clk::time_point t0 = clk::now();
			f();
			double s = std::chrono::duration<double>(clk::now() - t0).count();
			if (s < best)
				best = s;
		}
		return best;
	}

	std::set<layer_action> all_actions()
	{
		std::set<layer_action> a;
		a.insert(layer_action(layer_action::forward));
		a.insert(layer_action(layer_action::backward_data, 0));
		return a;
	}

	// Runs tester->run_forward_propagation for a single-input layer of shape [n][c][h][w].
	template <class Tester>
	double run_tester(float * y, const float * x, layer::const_ptr schema, layer_data::const_ptr data,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		const size_t bytes = (size_t)n * c * h * w * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, bytes);
		std::vector<plain_buffer::const_ptr> ins(1, make_buffer(x, bytes));
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		Tester tester;
		double s = timed(reps, [&]() {
			tester.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, data,
				layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(y, (const void *)(*out), bytes);
		return s;
	}

	template <class Updater>
	double run_updater_fwd(float * y, const float * x, layer::const_ptr schema, layer_data::const_ptr data,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		const size_t bytes = (size_t)n * c * h * w * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, bytes);
		std::vector<plain_buffer::const_ptr> ins(1, make_buffer(x, bytes));
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		Updater updater;
		std::set<layer_action> actions = all_actions();
		double s = timed(reps, [&]() {
			updater.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, data,
				layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
		});
		memcpy(y, (const void *)(*out), bytes);
		return s;
	}

	// Runs updater->run_backward_data_propagation. dx is read first when add_to_destination is set.
	template <class Updater>
	double run_updater_bwd(float * dx, const float * dy, const float * x_or_null, const float * y_or_null,
		layer::const_ptr schema, layer_data::const_ptr data,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int add_to_destination, int threads, int reps)
	{
		const size_t bytes = (size_t)n * c * h * w * sizeof(float);
		plain_buffer::ptr in_err = make_buffer(dx, bytes);
		plain_buffer::const_ptr out_err = make_buffer(dy, bytes);
		std::vector<plain_buffer::const_ptr> in_neurons(1, x_or_null ? make_buffer(x_or_null, bytes) : plain_buffer::ptr());
		plain_buffer::const_ptr out_neurons = y_or_null ? make_buffer(y_or_null, bytes) : plain_buffer::ptr();
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		Updater updater;
		std::set<layer_action> actions = all_actions();
		// With accumulation every repetition would add again, so the destination is restored each time.
		double s = timed(add_to_destination ? 1 : reps, [&]() {
			updater.run_backward_data_propagation(0, in_err, out_err, in_neurons, out_neurons, plain_buffer::ptr(), plain_buffer::ptr(),
				plain_buffer::ptr(), cfg, schema, data, layer_data_custom::const_ptr(), in_cfgs, out_cfg, add_to_destination != 0, actions, n);
		});
		memcpy(dx, (const void *)(*in_err), bytes);
		return s;
	}

	layer_data::ptr one_chunk(const float * v, unsigned int count)
	{
		layer_data::ptr d(new layer_data());
		d->push_back(std::vector<float>(v, v + count));
		return d;
	}
}

#define REF_GUARD_BEGIN try {
#define REF_GUARD_END } catch (const std::exception& e) { g_last_error = e.what(); return -1.0; }

extern "C"
{
	const char * ref_last_error() { return g_last_error.c_str(); }

	// nnforge/plain/batch_norm_layer_tester_plain.cpp:30-75
	double ref_bn_infer(float * y, const float * x, const float * gamma, const float * beta, const float * mean, const float * invsigma,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new batch_norm_layer(c));
		layer_data::ptr data(new layer_data());
		data->push_back(std::vector<float>(gamma, gamma + c));
		data->push_back(std::vector<float>(beta, beta + c));
		data->push_back(std::vector<float>(mean, mean + c));
		data->push_back(std::vector<float>(invsigma, invsigma + c));
		return run_tester<batch_norm_layer_tester_plain>(y, x, schema, data, n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/rectified_linear_layer_tester_plain.cpp:30-56
	double ref_relu_fwd(float * y, const float * x, float negative_slope, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new rectified_linear_layer(negative_slope));
		return run_tester<rectified_linear_layer_tester_plain>(y, x, schema, layer_data::const_ptr(), n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/rectified_linear_layer_updater_plain.cpp:62-107
	double ref_relu_bwd(float * dx, const float * dy, const float * x, float negative_slope, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new rectified_linear_layer(negative_slope));
		return run_updater_bwd<rectified_linear_layer_updater_plain>(dx, dy, x, 0, schema, layer_data::const_ptr(), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/parametric_rectified_linear_layer_tester_plain.cpp:30-71
	double ref_prelu_fwd(float * y, const float * x, const float * slope, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new parametric_rectified_linear_layer(c));
		return run_tester<parametric_rectified_linear_layer_tester_plain>(y, x, schema, one_chunk(slope, c), n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/parametric_rectified_linear_layer_updater_plain.cpp:74-135
	double ref_prelu_bwd_data(float * dx, const float * dy, const float * x, const float * slope, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new parametric_rectified_linear_layer(c));
		return run_updater_bwd<parametric_rectified_linear_layer_updater_plain>(dx, dy, x, 0, schema, one_chunk(slope, c), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/parametric_rectified_linear_layer_updater_plain.cpp:137-190; dslope is accumulated into.
	double ref_prelu_bwd_weights(float * dslope, const float * dy, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads)
	{
		REF_GUARD_BEGIN
		const size_t bytes = (size_t)n * c * h * w * sizeof(float);
		layer::const_ptr schema(new parametric_rectified_linear_layer(c));
		std::vector<plain_buffer::const_ptr> in_neurons(1, make_buffer(x, bytes));
		plain_buffer::const_ptr out_err = make_buffer(dy, bytes);
		layer_data::ptr gradient = one_chunk(dslope, c);
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		parametric_rectified_linear_layer_updater_plain updater;
		std::set<layer_action> actions = all_actions();
		double s = timed(1, [&]() {
			updater.run_backward_weights_propagation(in_neurons, out_err, plain_buffer::ptr(), plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema,
				gradient, layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
		});
		memcpy(dslope, &(*gradient)[0][0], c * sizeof(float));
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/exponential_linear_layer_tester_plain.cpp:30-54
	double ref_elu_fwd(float * y, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new exponential_linear_layer());
		return run_tester<exponential_linear_layer_tester_plain>(y, x, schema, layer_data::const_ptr(), n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/exponential_linear_layer_updater_plain.cpp:59-103 (derivative from the OUTPUT neurons)
	double ref_elu_bwd(float * dx, const float * dy, const float * y, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new exponential_linear_layer());
		return run_updater_bwd<exponential_linear_layer_updater_plain>(dx, dy, 0, y, schema, layer_data::const_ptr(), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/hyperbolic_tangent_layer_tester_plain.cpp:30-59
	double ref_tanh_fwd(float * y, const float * x, float scale, float steepness, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new hyperbolic_tangent_layer(scale, steepness));
		return run_tester<hyperbolic_tangent_layer_tester_plain>(y, x, schema, layer_data::const_ptr(), n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/hyperbolic_tangent_layer_updater_plain.cpp:62-112
	double ref_tanh_bwd(float * dx, const float * dy, const float * y, float scale, float steepness, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new hyperbolic_tangent_layer(scale, steepness));
		return run_updater_bwd<hyperbolic_tangent_layer_updater_plain>(dx, dy, 0, y, schema, layer_data::const_ptr(), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/sigmoid_layer_tester_plain.cpp:30-54
	double ref_sigmoid_fwd(float * y, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new sigmoid_layer());
		return run_tester<sigmoid_layer_tester_plain>(y, x, schema, layer_data::const_ptr(), n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/sigmoid_layer_updater_plain.cpp:59-103
	double ref_sigmoid_bwd(float * dx, const float * dy, const float * y, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new sigmoid_layer());
		return run_updater_bwd<sigmoid_layer_updater_plain>(dx, dy, 0, y, schema, layer_data::const_ptr(), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/softmax_layer_tester_plain.cpp:34-91
	double ref_softmax_fwd(float * y, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new softmax_layer());
		return run_tester<softmax_layer_tester_plain>(y, x, schema, layer_data::const_ptr(), n, c, h, w, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/softmax_layer_updater_plain.cpp:34-98 (forward of the training-side object)
	double ref_softmax_upd_fwd(float * y, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new softmax_layer());
		const size_t bytes = (size_t)n * c * h * w * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, bytes);
		std::vector<plain_buffer::const_ptr> ins(1, make_buffer(x, bytes));
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		softmax_layer_updater_plain updater;
		std::set<layer_action> actions = all_actions();
		// The scheduler sizes this scratch from the updater's own answer (one row of C floats per thread).
		plain_buffer::ptr working = make_buffer(0, updater.get_temporary_working_fixed_buffer_size(layer_action(layer_action::forward), actions, cfg, schema, in_cfgs, out_cfg));
		double s = timed(reps, [&]() {
			updater.run_forward_propagation(out, ins, working, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
				layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
		});
		memcpy(y, (const void *)(*out), bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/softmax_layer_updater_plain.cpp:100-166
	double ref_softmax_bwd(float * dx, const float * dy, const float * y, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new softmax_layer());
		return run_updater_bwd<softmax_layer_updater_plain>(dx, dy, 0, y, schema, layer_data::const_ptr(), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/add_layer_tester_plain.cpp:32-62
	double ref_add_fwd(float * y, const float * const * inputs, int input_count, float alpha, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int threads, int reps)
	{
		REF_GUARD_BEGIN
		const size_t bytes = (size_t)n * c * h * w * sizeof(float);
		layer::const_ptr schema(new add_layer(alpha));
		plain_buffer::ptr out = make_buffer(0, bytes);
		std::vector<plain_buffer::const_ptr> ins;
		for (int i = 0; i < input_count; ++i)
			ins.push_back(make_buffer(inputs[i], bytes));
		std::vector<layer_configuration_specific> in_cfgs(input_count, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		add_layer_tester_plain tester;
		double s = timed(reps, [&]() {
			tester.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
				layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(y, (const void *)(*out), bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/add_layer_updater_plain.cpp:66-109
	double ref_add_bwd(float * dx, const float * dy, float alpha, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		int add_to_destination, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new add_layer(alpha));
		return run_updater_bwd<add_layer_updater_plain>(dx, dy, 0, 0, schema, layer_data::const_ptr(), n, c, h, w, add_to_destination, threads, reps);
		REF_GUARD_END
	}

	// nnforge/plain/max_subsampling_layer_updater_plain.cpp:35-171. Output extents follow
	// nnforge/max_subsampling_layer.cpp:125-133 and are returned through out_h / out_w.
	// argmax receives the absolute input element offsets (unsigned int), as the plain backend stores them.
	double ref_maxpool_fwd(float * y, unsigned int * argmax, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		unsigned int win_w, unsigned int win_h, unsigned int stride_w, unsigned int stride_h, int is_min,
		unsigned int * out_h, unsigned int * out_w, int threads, int reps)
	{
		REF_GUARD_BEGIN
		std::vector<unsigned int> sizes; sizes.push_back(win_w); sizes.push_back(win_h);
		std::vector<unsigned int> strides; strides.push_back(stride_w); strides.push_back(stride_h);
		std::vector<bool> round_ups(2, false);
		std::shared_ptr<max_subsampling_layer> l(new max_subsampling_layer(sizes, 1, 1, is_min != 0, false, round_ups, strides));
		layer::const_ptr schema = l;
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = l->get_output_layer_configuration_specific(in_cfgs);
		*out_w = out_cfg.dimension_sizes[0];
		*out_h = out_cfg.dimension_sizes[1];
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * out_cfg.get_neuron_count() * sizeof(float);
		if (!y)
			return 0.0; // shape query only
		plain_buffer::ptr out = make_buffer(0, out_bytes);
		plain_buffer::ptr idx = make_buffer(0, out_bytes);
		std::vector<plain_buffer::const_ptr> ins(1, make_buffer(x, in_bytes));
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		max_subsampling_layer_updater_plain updater;
		std::set<layer_action> actions = all_actions();
		double s = timed(reps, [&]() {
			updater.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), idx, cfg, schema, layer_data::const_ptr(),
				layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
		});
		memcpy(y, (const void *)(*out), out_bytes);
		if (argmax)
			memcpy(argmax, (const void *)(*idx), out_bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/max_subsampling_layer_tester_plain.cpp:170-288 (inference-side object, value only)
	double ref_maxpool_tester_fwd(float * y, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		unsigned int win_w, unsigned int win_h, unsigned int stride_w, unsigned int stride_h, int is_min, int threads, int reps)
	{
		REF_GUARD_BEGIN
		std::vector<unsigned int> sizes; sizes.push_back(win_w); sizes.push_back(win_h);
		std::vector<unsigned int> strides; strides.push_back(stride_w); strides.push_back(stride_h);
		std::vector<bool> round_ups(2, false);
		std::shared_ptr<max_subsampling_layer> l(new max_subsampling_layer(sizes, 1, 1, is_min != 0, false, round_ups, strides));
		layer::const_ptr schema = l;
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = l->get_output_layer_configuration_specific(in_cfgs);
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * out_cfg.get_neuron_count() * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, out_bytes);
		std::vector<plain_buffer::const_ptr> ins(1, make_buffer(x, in_bytes));
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		max_subsampling_layer_tester_plain tester;
		double s = timed(reps, [&]() {
			tester.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
				layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(y, (const void *)(*out), out_bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/max_subsampling_layer_updater_plain.cpp:173-231. With threads == 1 and
	// add_to_destination != 0 onto a zeroed dx this is the deterministic "sum of contributions in
	// ascending output index" that overlapping windows need (the non-accumulating branch overwrites).
	double ref_maxpool_bwd(float * dx, const float * dy, const unsigned int * argmax, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		unsigned int out_h, unsigned int out_w, int add_to_destination, int threads)
	{
		REF_GUARD_BEGIN
		std::vector<unsigned int> sizes(2, 1);
		std::shared_ptr<max_subsampling_layer> l(new max_subsampling_layer(sizes, 1, 1, false, false, std::vector<bool>(2, false), std::vector<unsigned int>(2, 1)));
		layer::const_ptr schema = l;
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, out_h, out_w);
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * c * out_h * out_w * sizeof(float);
		plain_buffer::ptr in_err = make_buffer(dx, in_bytes);
		plain_buffer::const_ptr out_err = make_buffer(dy, out_bytes);
		plain_buffer::ptr idx = make_buffer(argmax, out_bytes);
		std::vector<plain_buffer::const_ptr> in_neurons(1, plain_buffer::ptr());
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		max_subsampling_layer_updater_plain updater;
		std::set<layer_action> actions = all_actions();
		double s = timed(1, [&]() {
			updater.run_backward_data_propagation(0, in_err, out_err, in_neurons, plain_buffer::const_ptr(), plain_buffer::ptr(), plain_buffer::ptr(),
				idx, cfg, schema, layer_data::const_ptr(), layer_data_custom::const_ptr(), in_cfgs, out_cfg, add_to_destination != 0, actions, n);
		});
		memcpy(dx, (const void *)(*in_err), in_bytes);
		return s;
		REF_GUARD_END
	}
	// nnforge/plain/negative_log_likelihood_layer_tester_plain.cpp:30-92 (updater == 0) or
	// negative_log_likelihood_layer_updater_plain.cpp:30-92 (updater != 0): err[n][1][h][w] from predicted and
	// actual [n][c][h][w] and an optional scale mask [n][1][h][w].
	double ref_nll_fwd(float * err, const float * predicted, const float * actual, const float * mask_or_null, float scale,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int updater, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new negative_log_likelihood_layer(scale));
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * h * w * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, out_bytes);
		std::vector<plain_buffer::const_ptr> ins;
		ins.push_back(make_buffer(predicted, in_bytes));
		ins.push_back(make_buffer(actual, in_bytes));
		std::vector<layer_configuration_specific> in_cfgs(2, make_config(c, h, w));
		if (mask_or_null)
		{
			ins.push_back(make_buffer(mask_or_null, out_bytes));
			in_cfgs.push_back(make_config(1, h, w));
		}
		layer_configuration_specific out_cfg = make_config(1, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions = all_actions();
		negative_log_likelihood_layer_tester_plain tester;
		negative_log_likelihood_layer_updater_plain upd;
		double s = timed(reps, [&]() {
			if (updater)
				upd.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
			else
				tester.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(err, (const void *)(*out), out_bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/negative_log_likelihood_layer_updater_plain.cpp:94-158: gradient with respect to the predictions
	// (input 0); the layer is a loss, its output errors are not read.
	double ref_nll_bwd(float * dpredicted, const float * predicted, const float * actual, const float * mask_or_null, float scale,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int add_to_destination, int threads)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new negative_log_likelihood_layer(scale));
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * h * w * sizeof(float);
		plain_buffer::ptr in_err = make_buffer(dpredicted, in_bytes);
		std::vector<plain_buffer::const_ptr> ins;
		ins.push_back(make_buffer(predicted, in_bytes));
		ins.push_back(make_buffer(actual, in_bytes));
		std::vector<layer_configuration_specific> in_cfgs(2, make_config(c, h, w));
		if (mask_or_null)
		{
			ins.push_back(make_buffer(mask_or_null, out_bytes));
			in_cfgs.push_back(make_config(1, h, w));
		}
		layer_configuration_specific out_cfg = make_config(1, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions = all_actions();
		negative_log_likelihood_layer_updater_plain upd;
		double s = timed(1, [&]() {
			upd.run_backward_data_propagation(0, in_err, plain_buffer::const_ptr(), ins, plain_buffer::const_ptr(), plain_buffer::ptr(), plain_buffer::ptr(),
				plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(), layer_data_custom::const_ptr(), in_cfgs, out_cfg, add_to_destination != 0, actions, n);
		});
		memcpy(dpredicted, (const void *)(*in_err), in_bytes);
		return s;
		REF_GUARD_END
	}
	// nnforge/plain/cross_entropy_layer_tester_plain.cpp:32-98 (updater == 0) or cross_entropy_layer_updater_plain.cpp:32-101
	// (updater != 0): err[n][1][h][w] from predicted and actual [n][c][h][w] and an optional scale mask [n][1][h][w].
	double ref_cross_entropy_fwd(float * err, const float * predicted, const float * actual, const float * mask_or_null, float scale,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int updater, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new cross_entropy_layer(scale));
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * h * w * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, out_bytes);
		std::vector<plain_buffer::const_ptr> ins;
		ins.push_back(make_buffer(predicted, in_bytes));
		ins.push_back(make_buffer(actual, in_bytes));
		std::vector<layer_configuration_specific> in_cfgs(2, make_config(c, h, w));
		if (mask_or_null)
		{
			ins.push_back(make_buffer(mask_or_null, out_bytes));
			in_cfgs.push_back(make_config(1, h, w));
		}
		layer_configuration_specific out_cfg = make_config(1, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions = all_actions();
		cross_entropy_layer_tester_plain tester;
		cross_entropy_layer_updater_plain upd;
		double s = timed(reps, [&]() {
			if (updater)
				upd.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
			else
				tester.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(err, (const void *)(*out), out_bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/cross_entropy_layer_updater_plain.cpp:103-175: the plain backend's backward action as it is (it stores
	// zeros: the gradient is computed into a variable that shadows the one that is stored, :150-168).
	double ref_cross_entropy_bwd(float * dpredicted, const float * predicted, const float * actual, const float * mask_or_null, float scale,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int add_to_destination, int threads)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new cross_entropy_layer(scale));
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * h * w * sizeof(float);
		plain_buffer::ptr in_err = make_buffer(dpredicted, in_bytes);
		std::vector<plain_buffer::const_ptr> ins;
		ins.push_back(make_buffer(predicted, in_bytes));
		ins.push_back(make_buffer(actual, in_bytes));
		std::vector<layer_configuration_specific> in_cfgs(2, make_config(c, h, w));
		if (mask_or_null)
		{
			ins.push_back(make_buffer(mask_or_null, out_bytes));
			in_cfgs.push_back(make_config(1, h, w));
		}
		layer_configuration_specific out_cfg = make_config(1, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions = all_actions();
		cross_entropy_layer_updater_plain upd;
		double s = timed(1, [&]() {
			upd.run_backward_data_propagation(0, in_err, plain_buffer::const_ptr(), ins, plain_buffer::const_ptr(), plain_buffer::ptr(), plain_buffer::ptr(),
				plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(), layer_data_custom::const_ptr(), in_cfgs, out_cfg, add_to_destination != 0, actions, n);
		});
		memcpy(dpredicted, (const void *)(*in_err), in_bytes);
		return s;
		REF_GUARD_END
	}
	// nnforge/plain/accuracy_layer_tester_plain.cpp:30-112 (updater == 0) or accuracy_layer_updater_plain.cpp (updater != 0):
	// out[n][top_n + 1][h][w] from predicted and actual [n][c][h][w] and an optional mask [n][1][h][w].
	double ref_accuracy_fwd(float * out, const float * predicted, const float * actual, const float * mask_or_null, unsigned int top_n,
		unsigned int n, unsigned int c, unsigned int h, unsigned int w, int updater, int threads, int reps)
	{
		REF_GUARD_BEGIN
		layer::const_ptr schema(new accuracy_layer(top_n));
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t mask_bytes = (size_t)n * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * (top_n + 1) * h * w * sizeof(float);
		plain_buffer::ptr outb = make_buffer(0, out_bytes);
		std::vector<plain_buffer::const_ptr> ins;
		ins.push_back(make_buffer(predicted, in_bytes));
		ins.push_back(make_buffer(actual, in_bytes));
		std::vector<layer_configuration_specific> in_cfgs(2, make_config(c, h, w));
		if (mask_or_null)
		{
			ins.push_back(make_buffer(mask_or_null, mask_bytes));
			in_cfgs.push_back(make_config(1, h, w));
		}
		layer_configuration_specific out_cfg = make_config(top_n + 1, h, w);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions;
		actions.insert(layer_action(layer_action::forward));
		accuracy_layer_tester_plain tester;
		accuracy_layer_updater_plain upd;
		double s = timed(reps, [&]() {
			if (updater)
				upd.run_forward_propagation(outb, ins, plain_buffer::ptr(), plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
			else
				tester.run_forward_propagation(outb, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(out, (const void *)(*outb), out_bytes);
		return s;
		REF_GUARD_END
	}
	// nnforge/plain/average_subsampling_layer_tester_plain.cpp:30-148 (updater == 0) or the updater's forward
	// (average_subsampling_layer_updater_plain.cpp:30-148): windows win_w x win_h, stride = window, default alpha.
	double ref_avgpool_fwd(float * y, const float * x, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		unsigned int win_w, unsigned int win_h, int updater, int threads, int reps)
	{
		REF_GUARD_BEGIN
		std::vector<average_subsampling_factor> sizes;
		sizes.push_back(average_subsampling_factor(win_w));
		sizes.push_back(average_subsampling_factor(win_h));
		layer::const_ptr schema(new average_subsampling_layer(sizes));
		const unsigned int oh = h / win_h, ow = w / win_w;
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * c * oh * ow * sizeof(float);
		plain_buffer::ptr out = make_buffer(0, out_bytes);
		std::vector<plain_buffer::const_ptr> ins(1, make_buffer(x, in_bytes));
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, oh, ow);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions = all_actions();
		average_subsampling_layer_tester_plain tester;
		average_subsampling_layer_updater_plain upd;
		double s = timed(reps, [&]() {
			if (updater)
				upd.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, actions, n);
			else
				tester.run_forward_propagation(out, ins, plain_buffer::ptr(), plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(),
					layer_data_custom::const_ptr(), in_cfgs, out_cfg, n);
		});
		memcpy(y, (const void *)(*out), out_bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/plain/average_subsampling_layer_updater_plain.cpp:151-297
	double ref_avgpool_bwd(float * dx, const float * dy, unsigned int n, unsigned int c, unsigned int h, unsigned int w,
		unsigned int win_w, unsigned int win_h, int add_to_destination, int threads)
	{
		REF_GUARD_BEGIN
		std::vector<average_subsampling_factor> sizes;
		sizes.push_back(average_subsampling_factor(win_w));
		sizes.push_back(average_subsampling_factor(win_h));
		layer::const_ptr schema(new average_subsampling_layer(sizes));
		const unsigned int oh = h / win_h, ow = w / win_w;
		const size_t in_bytes = (size_t)n * c * h * w * sizeof(float);
		const size_t out_bytes = (size_t)n * c * oh * ow * sizeof(float);
		plain_buffer::ptr in_err = make_buffer(dx, in_bytes);
		plain_buffer::const_ptr out_err = make_buffer(dy, out_bytes);
		std::vector<plain_buffer::const_ptr> in_neurons(1, plain_buffer::ptr());
		std::vector<layer_configuration_specific> in_cfgs(1, make_config(c, h, w));
		layer_configuration_specific out_cfg = make_config(c, oh, ow);
		plain_running_configuration::const_ptr cfg = make_running_config(threads);
		std::set<layer_action> actions = all_actions();
		average_subsampling_layer_updater_plain upd;
		double s = timed(1, [&]() {
			upd.run_backward_data_propagation(0, in_err, out_err, in_neurons, plain_buffer::const_ptr(), plain_buffer::ptr(), plain_buffer::ptr(),
				plain_buffer::ptr(), cfg, schema, layer_data::const_ptr(), layer_data_custom::const_ptr(), in_cfgs, out_cfg, add_to_destination != 0, actions, n);
		});
		memcpy(dx, (const void *)(*in_err), in_bytes);
		return s;
		REF_GUARD_END
	}

	// nnforge/stat_data_bunch_writer.cpp:44-111: stats[4][c] = {min, max, average, std_dev} of y[n][c][hw], entries fed one by
	// one as forward_propagation hands them to the writer
	double ref_feature_map_stats(float * stats, const float * y, unsigned int n, unsigned int c, unsigned int h, unsigned int w)
	{
		REF_GUARD_BEGIN
		stat_data_bunch_writer writer;
		std::map<std::string, layer_configuration_specific> cfg;
		cfg.insert(std::make_pair(std::string("bn"), make_config(c, h, w)));
		writer.set_config_map(cfg);
		const size_t per_entry = (size_t)c * h * w;
		for (unsigned int e = 0; e < n; ++e)
		{
			std::map<std::string, const float *> data;
			data.insert(std::make_pair(std::string("bn"), y + e * per_entry));
			writer.write(e, data);
		}
		const std::vector<feature_map_data_stat> st = writer.get_stat().find("bn")->second;
		for (unsigned int ch = 0; ch < c; ++ch)
		{
			stats[ch] = st[ch].min;
			stats[c + ch] = st[ch].max;
			stats[2 * c + ch] = st[ch].average;
			stats[3 * c + ch] = st[ch].std_dev;
		}
		return 0.0;
		REF_GUARD_END
	}
}
