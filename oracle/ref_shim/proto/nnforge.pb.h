// Stand-in for the protobuf-generated accessors that the nnForge layer classes of this path touch in their
// read_proto / write_proto members (BatchNorm, ReLU, PReLU, TanH, Add, MaxSubsampling, NegativeLogLikelihood, CrossEntropy, Accuracy, AverageSubsampling;
// the other hot-path layers have no parameters). protoc is not available where the oracle is built and
// the oracle never (de)serialises a schema, so these are plain structs with the same accessor names.
// Test infrastructure only.
#pragma once
#include <string>
#include <vector>

namespace nnforge
{
	namespace protobuf
	{
#define NNF_SHIM_FIELD(type, name) \
		private: type name##_{}; bool has_##name##_ = false; \
		public: type name() const { return name##_; } \
		bool has_##name() const { return has_##name##_; } \
		void set_##name(type v) { name##_ = v; has_##name##_ = true; }

#define NNF_SHIM_MESSAGE(type, name) \
		private: type name##_; bool has_##name##_ = false; \
		public: const type& name() const { return name##_; } \
		bool has_##name() const { return has_##name##_; } \
		type * mutable_##name() { has_##name##_ = true; return &name##_; }

		class ReLUParam { NNF_SHIM_FIELD(float, negative_slope) };
		class BatchNormParam { NNF_SHIM_FIELD(unsigned int, feature_map_count) NNF_SHIM_FIELD(float, epsilon) };
		class AddParam { NNF_SHIM_FIELD(float, alpha) };
		class TanHParam { NNF_SHIM_FIELD(float, scale) NNF_SHIM_FIELD(float, steepness) };
		class PReLUParam { NNF_SHIM_FIELD(unsigned int, feature_map_count) };
		class NegativeLogLikelihoodParam { NNF_SHIM_FIELD(float, scale) };
		class CrossEntropyParam { NNF_SHIM_FIELD(float, scale) };
		class AccuracyParam { NNF_SHIM_FIELD(unsigned int, top_n) };

		enum MaxSubsamplingParam_MaxFunction { MaxSubsamplingParam_MaxFunction_MAX = 0, MaxSubsamplingParam_MaxFunction_MIN = 1 };
		class MaxSubsamplingParam_MaxSubsamplingDimensionParam
		{
			NNF_SHIM_FIELD(unsigned int, subsampling_size) NNF_SHIM_FIELD(bool, round_up) NNF_SHIM_FIELD(unsigned int, stride)
		};
		class MaxSubsamplingParam_MaxSubsamplingFeatureMapParam { NNF_SHIM_FIELD(unsigned int, subsampling_size) };
		class MaxSubsamplingParam_MaxSubsamplingEntryParam { NNF_SHIM_FIELD(unsigned int, subsampling_size) };
		class MaxSubsamplingParam
		{
			NNF_SHIM_FIELD(bool, tiling)
			NNF_SHIM_FIELD(MaxSubsamplingParam_MaxFunction, function)
			NNF_SHIM_MESSAGE(MaxSubsamplingParam_MaxSubsamplingFeatureMapParam, feature_map_param)
			NNF_SHIM_MESSAGE(MaxSubsamplingParam_MaxSubsamplingEntryParam, entry_param)
		private:
			std::vector<MaxSubsamplingParam_MaxSubsamplingDimensionParam> dims_;
		public:
			int dimension_param_size() const { return static_cast<int>(dims_.size()); }
			const MaxSubsamplingParam_MaxSubsamplingDimensionParam& dimension_param(int i) const { return dims_[i]; }
			MaxSubsamplingParam_MaxSubsamplingDimensionParam * add_dimension_param() { dims_.emplace_back(); return &dims_.back(); }
		};

		class AverageSubsamplingParam_AverageSubsamplingDimensionParam
		{
			NNF_SHIM_FIELD(unsigned int, subsampling_size) NNF_SHIM_FIELD(unsigned int, subsampled_size)
		};
		class AverageSubsamplingParam_AverageSubsamplingFeatureMapParam
		{
			NNF_SHIM_FIELD(unsigned int, subsampling_size) NNF_SHIM_FIELD(unsigned int, subsampled_size)
		};
		class AverageSubsamplingParam_AverageSubsamplingEntryParam { NNF_SHIM_FIELD(unsigned int, subsampling_size) };
		class AverageSubsamplingParam
		{
			NNF_SHIM_FIELD(float, alpha)
			NNF_SHIM_MESSAGE(AverageSubsamplingParam_AverageSubsamplingFeatureMapParam, feature_map_param)
			NNF_SHIM_MESSAGE(AverageSubsamplingParam_AverageSubsamplingEntryParam, entry_param)
		private:
			std::vector<AverageSubsamplingParam_AverageSubsamplingDimensionParam> dims_;
		public:
			int dimension_param_size() const { return static_cast<int>(dims_.size()); }
			const AverageSubsamplingParam_AverageSubsamplingDimensionParam& dimension_param(int i) const { return dims_[i]; }
			AverageSubsamplingParam_AverageSubsamplingDimensionParam * add_dimension_param() { dims_.emplace_back(); return &dims_.back(); }
		};

		class Layer
		{
			NNF_SHIM_MESSAGE(ReLUParam, relu_param)
			NNF_SHIM_MESSAGE(BatchNormParam, batch_norm_param)
			NNF_SHIM_MESSAGE(AddParam, add_param)
			NNF_SHIM_MESSAGE(TanHParam, tanh_param)
			NNF_SHIM_MESSAGE(PReLUParam, prelu_param)
			NNF_SHIM_MESSAGE(NegativeLogLikelihoodParam, negative_log_likelihood_param)
			NNF_SHIM_MESSAGE(CrossEntropyParam, cross_entropy_param)
			NNF_SHIM_MESSAGE(AccuracyParam, accuracy_param)
			NNF_SHIM_MESSAGE(AverageSubsamplingParam, average_subsampling_param)
			NNF_SHIM_MESSAGE(MaxSubsamplingParam, max_subsampling_param)
		private:
			std::string type_;
		public:
			const std::string& type() const { return type_; }
		};
#undef NNF_SHIM_FIELD
#undef NNF_SHIM_MESSAGE
	}
}
