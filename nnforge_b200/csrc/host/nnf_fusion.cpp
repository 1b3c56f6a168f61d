#include "nnf_fusion.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <sstream>

namespace nnf_b200
{
	namespace
	{
		bool is_act(const std::string& t)
		{
			return t == "ReLU" || t == "PReLU" || t == "ELU" || t == "TanH" || t == "Sigmoid";
		}

		bool spatial_pool_2d(const layer& l)
		{
			return l.subsampling_sizes.size() == 2 && l.feature_map_subsampling_size == 1 && l.entry_subsampling_size == 1 && !l.tiling;
		}

		struct graph
		{
			const std::vector<schema_node>& nodes;
			std::map<std::string, int> index;
			std::vector<std::vector<int>> readers;

			explicit graph(const std::vector<schema_node>& n) : nodes(n), readers(n.size())
			{
				for (size_t i = 0; i < n.size(); ++i)
				{
					if (index.count(n[i].name))
						throw neural_network_exception("Duplicate layer name in schema: " + n[i].name);
					index[n[i].name] = (int)i;
				}
				for (size_t i = 0; i < n.size(); ++i)
					for (const std::string& in : n[i].inputs)
					{
						auto it = index.find(in);
						if (it == index.end())
							continue; // a data layer outside the list
						if (it->second >= (int)i)
							throw neural_network_exception("Schema is not in execution order at layer " + n[i].name);
						readers[it->second].push_back((int)i);
					}
			}

			// the only reader of node i, when its output can stay inside a fused kernel; else -1
			int sole_reader(int i) const
			{
				return (!nodes[i].output_needed && readers[i].size() == 1) ? readers[i][0] : -1;
			}

			// a reader of node i of the given type, whatever else reads it; else -1
			int reader_of_type(int i, const std::string& type) const
			{
				for (int r : readers[i])
					if (nodes[r].params.type_name == type)
						return r;
				return -1;
			}
		};
	}

	std::vector<fused_group> plan_fusion(const std::vector<schema_node>& nodes, bool training)
	{
		const graph g(nodes);
		std::vector<bool> taken(nodes.size(), false);
		std::vector<fused_group> plan;
		for (int i = 0; i < (int)nodes.size(); ++i)
		{
			if (taken[i])
				continue;
			const std::string& type = nodes[i].params.type_name;
			fused_group grp;
			grp.members.push_back(i);

			if (type == "Softmax")
			{
				grp.softmax = i;
				// the loss must read the probabilities as its first input; other readers of the probabilities are fine
				const int loss = g.reader_of_type(i, "NegativeLogLikelihood");
				if (loss >= 0 && !taken[loss] && !nodes[loss].inputs.empty() && nodes[loss].inputs[0] == nodes[i].name)
				{
					// everything the loss reads besides the probabilities must already exist when the softmax runs
					bool ready = true;
					for (size_t k = 1; k < nodes[loss].inputs.size(); ++k)
					{
						auto it = g.index.find(nodes[loss].inputs[k]);
						if (it != g.index.end() && it->second > i)
							ready = false;
					}
					if (ready)
					{
						grp.kind = fused_softmax_nll;
						grp.loss = loss;
						grp.members.push_back(loss);
						grp.entry_point = "nnf_softmax_nll_fwd";
					}
				}
			}
			else if (training && type == "BatchNorm")
			{
				grp.bn = i;
				int cur = i, prelus = 0;
				while (grp.acts.size() < 2)
				{
					const int next = g.sole_reader(cur);
					if (next < 0 || taken[next] || !is_act(nodes[next].params.type_name) || nodes[next].inputs.size() != 1)
						break;
					if (nodes[next].params.type_name == "PReLU" && ++prelus > 1)
						break;
					grp.acts.push_back(next);
					grp.members.push_back(next);
					cur = next;
				}
				if (!grp.acts.empty())
				{
					grp.kind = fused_bn_train_act;
					grp.entry_point = "nnf_bn_train_fwd";
				}
			}
			else if (!training && (type == "BatchNorm" || type == "Add" || is_act(type)))
			{
				int cur = i;
				if (type == "BatchNorm")
					grp.bn = i;
				auto try_add = [&](int node, int from) -> bool
				{
					// an Add of exactly two inputs, one of which is the running chain; the other becomes the residual
					const schema_node& a = nodes[node];
					if (a.params.type_name != "Add" || a.inputs.size() != 2)
						return false;
					const std::string& me = nodes[from].name;
					if ((a.inputs[0] == me) == (a.inputs[1] == me))
						return false; // neither, or both
					const std::string& other = a.inputs[0] == me ? a.inputs[1] : a.inputs[0];
					auto it = g.index.find(other);
					if (it != g.index.end() && it->second > i && !taken[it->second])
						return false; // the residual is produced after the head of the chain: it would not exist yet
					grp.add = node;
					grp.residual_input = other;
					return true;
				};
				if (type == "Add")
				{
					// a bare Add heads the chain only in its two-input form; the kernel treats input 0 as x, input 1 as residual
					if (nodes[i].inputs.size() == 2)
					{
						grp.add = i;
						grp.residual_input = nodes[i].inputs[1];
					}
				}
				else if (is_act(type))
					grp.acts.push_back(i);
				if (grp.bn >= 0)
				{
					const int next = g.sole_reader(cur);
					if (next >= 0 && !taken[next] && try_add(next, cur))
					{
						grp.members.push_back(next);
						cur = next;
					}
				}
				if (type != "Add" || grp.add >= 0)
				{
					int prelus = (is_act(type) && type == "PReLU") ? 1 : 0;
					while (grp.acts.size() < 2)
					{
						const int next = g.sole_reader(cur);
						if (next < 0 || taken[next] || !is_act(nodes[next].params.type_name) || nodes[next].inputs.size() != 1)
							break;
						if (nodes[next].params.type_name == "PReLU" && ++prelus > 1)
							break;
						grp.acts.push_back(next);
						grp.members.push_back(next);
						cur = next;
					}
				}
				// BN / Add -> exactly one ReLU -> pooling: the pooled kernels write the ReLU output themselves, so it may
				// have other readers; they implement an Add with alpha 1 only
				const bool relu_tail = grp.acts.size() == 1 && nodes[grp.acts[0]].params.type_name == "ReLU" && (grp.bn >= 0 || grp.add >= 0)
					&& (grp.add < 0 || nodes[grp.add].params.alpha == 1.0F);
				if (relu_tail)
				{
					int pool = g.reader_of_type(cur, "MaxSubsampling");
					fused_kind kind = fused_bn_add_relu_maxpool;
					const char * entry = "nnf_bn_add_relu_maxpool_fwd";
					if (pool < 0)
					{
						pool = g.reader_of_type(cur, "AverageSubsampling");
						kind = fused_bn_add_relu_avgpool;
						entry = "nnf_bn_add_relu_avgpool_fwd";
					}
					if (pool >= 0 && !taken[pool] && nodes[pool].inputs.size() == 1 && spatial_pool_2d(nodes[pool].params))
					{
						grp.kind = kind;
						grp.pool = pool;
						grp.members.push_back(pool);
						grp.entry_point = entry;
					}
				}
				if (grp.kind == fused_single_layer && grp.members.size() > 1)
				{
					grp.kind = fused_bn_act;
					grp.entry_point = "nnf_bn_infer_act";
				}
			}

			for (int m : grp.members)
				taken[m] = true;
			// outputs that stay inside the kernel: every member but the last, except the tensors the fused kernels write
			// anyway (the ReLU output of the pooled forms, the probabilities of softmax + loss)
			for (size_t k = 0; k + 1 < grp.members.size(); ++k)
			{
				const int m = grp.members[k];
				const bool written = ((grp.kind == fused_bn_add_relu_maxpool || grp.kind == fused_bn_add_relu_avgpool) && m == grp.acts[0])
					|| (grp.kind == fused_softmax_nll && m == grp.softmax);
				if (!written)
					grp.elided.push_back(m);
			}
			plan.push_back(grp);
		}
		return plan;
	}
}

namespace nnf_b200
{
	buffer_plan plan_forward_buffers(const std::vector<schema_node>& nodes, const std::vector<fused_group>& groups,
		const std::vector<int>& can_write, const std::vector<size_t>& bytes)
	{
		const int n = (int)nodes.size();
		if ((int)can_write.size() != n || (int)bytes.size() != n)
			throw neural_network_exception("plan_forward_buffers: one answer and one size per node expected");
		std::map<std::string, int> index;
		for (int i = 0; i < n; ++i)
			index[nodes[i].name] = i;
		// per node: the action (position) that writes its output, the action that runs it, whether its output exists, and which
		// inputs the RUNNING object of its group reads from outside the group
		std::vector<int> written_at(n), runs_at(n), head_of(n);
		std::vector<bool> exists(n, true), is_head(n, false);
		for (const fused_group& g : groups)
		{
			const int head = g.members.at(0);
			is_head[head] = true;
			for (int m : g.members)
			{
				written_at[m] = head;
				runs_at[m] = head;
				head_of[m] = head;
			}
			for (int e : g.elided)
				exists[e] = false;
		}
		// last action that reads each output
		std::vector<int> last_read(n, -1);
		for (int i = 0; i < n; ++i)
			for (const std::string& in : nodes[i].inputs)
			{
				auto it = index.find(in);
				if (it == index.end())
					continue;                               // a data layer: not planned here
				if (head_of[it->second] == head_of[i] && !is_head[i] && !exists[it->second])
					continue;                               // a link inside a fused group: never materialised, never read
				last_read[it->second] = std::max(last_read[it->second], runs_at[i]);
			}
		for (int i = 0; i < n; ++i)
			if (nodes[i].output_needed)
				last_read[i] = n;                           // a network output stays to the end
		buffer_plan plan;
		plan.buffer_of_node.assign(n, -1);
		plan.written_in_place.assign(n, -1);
		std::vector<int> free_at;                          // per buffer: the first action at which it is free again
		for (int a = 0; a < n; ++a)                        // actions in order; a group's outputs are all written at its head
		{
			if (!is_head[a])
				continue;
			const fused_group * grp = nullptr;
			for (const fused_group& g : groups)
				if (g.members.at(0) == a)
					grp = &g;
			std::vector<int> outputs;
			for (int m : grp->members)
				if (exists[m])
					outputs.push_back(m);
			bool first_output = true;
			for (int o : outputs)
			{
				int chosen = -1;
				// in place over an input of the running object: the group's own input for a head
				if (first_output && can_write[a] >= 0 && can_write[a] < (int)nodes[a].inputs.size())
				{
					auto it = index.find(nodes[a].inputs[can_write[a]]);
					if (it != index.end() && exists[it->second] && last_read[it->second] == a && plan.buffer_of_node[it->second] >= 0
						&& plan.buffer_bytes_per_entry[plan.buffer_of_node[it->second]] >= bytes[o])
					{
						chosen = plan.buffer_of_node[it->second];
						plan.written_in_place[o] = can_write[a];
					}
				}
				first_output = false;
				if (chosen < 0)
				{
					for (size_t b = 0; b < free_at.size(); ++b)
						if (free_at[b] <= a && plan.buffer_bytes_per_entry[b] >= bytes[o]
							&& (chosen < 0 || plan.buffer_bytes_per_entry[b] < plan.buffer_bytes_per_entry[chosen]))
							chosen = (int)b;
				}
				if (chosen < 0)
				{
					chosen = (int)free_at.size();
					free_at.push_back(0);
					plan.buffer_bytes_per_entry.push_back(bytes[o]);
				}
				plan.buffer_of_node[o] = chosen;
				// an output nobody reads is still written: it keeps its buffer through its own action
				free_at[chosen] = std::max(last_read[o], a) + 1;
			}
		}
		for (size_t b : plan.buffer_bytes_per_entry)
			plan.total_bytes_per_entry += b;
		return plan;
	}
}

namespace nnf_b200
{
	namespace
	{
		std::vector<std::string> split(const std::string& s, char sep)
		{
			std::vector<std::string> out;
			std::stringstream ss(s);
			std::string item;
			while (std::getline(ss, item, sep))
				if (!item.empty())
					out.push_back(item);
			return out;
		}

		std::vector<unsigned int> sizes(const std::string& val)
		{
			std::vector<unsigned int> r;
			for (const std::string& v : split(val, 'x'))
				r.push_back((unsigned int)std::stoul(v));
			return r;
		}
	}

	std::vector<schema_node> parse_schema(const std::string& spec)
	{
		std::vector<schema_node> nodes;
		for (const std::string& line : split(spec, '\n'))
		{
			const std::vector<std::string> tok = split(line, ' ');
			if (tok.size() < 3)
				throw neural_network_exception("Bad schema line: " + line);
			schema_node n;
			n.name = tok[0];
			n.params.type_name = tok[1];
			n.params.instance_name = tok[0];
			if (tok[2] != "-")
				n.inputs = split(tok[2], ',');
			for (size_t k = 3; k < tok.size(); ++k)
			{
				if (tok[k] == "needed") { n.output_needed = true; continue; }
				if (tok[k] == "min") { n.params.is_min = true; continue; }
				const size_t eq = tok[k].find('=');
				if (eq == std::string::npos)
					throw neural_network_exception("Bad schema token: " + tok[k]);
				const std::string key = tok[k].substr(0, eq), val = tok[k].substr(eq + 1);
				if (key == "alpha") n.params.alpha = std::stof(val);
				else if (key == "slope") n.params.negative_slope = std::stof(val);
				else if (key == "scale") n.params.scale = std::stof(val);
				else if (key == "steepness") n.params.steepness = std::stof(val);
				else if (key == "eps") n.params.epsilon = std::stof(val);
				else if (key == "topn") n.params.top_n = (unsigned int)std::stoul(val);
				else if (key == "win") n.params.subsampling_sizes = sizes(val);
				else if (key == "stride") n.params.strides = sizes(val);
				else if (key == "roundup")
				{
					n.params.round_ups.clear();
					for (unsigned int v : sizes(val))
						n.params.round_ups.push_back(v != 0);
				}
				else if (key == "fm") n.params.feature_map_subsampling_size = (unsigned int)std::stoul(val);
				else if (key == "tiling") n.params.tiling = val != "0";
				else throw neural_network_exception("Unknown schema key: " + key);
			}
			nodes.push_back(n);
		}
		return nodes;
	}
}

// ---- flat driver for tests -------------------------------------------------------------------------
// spec: the text form of parse_schema.
// result: one group per line, "kind entry_point members=a,b,c residual=name elided=a,b".
using namespace nnf_b200;

namespace
{
	std::string g_fusion_error;
}

extern "C" __attribute__((visibility("default"))) const char * nnfh_fusion_last_error() { return g_fusion_error.c_str(); }

extern "C" __attribute__((visibility("default"))) int nnfh_plan_fusion(const char * spec, int training, char * out, size_t out_size)
{
	try
	{
		const std::vector<schema_node> nodes = parse_schema(spec);
		static const char * kKinds[] = {"single", "bn_act", "bn_add_relu_maxpool", "bn_add_relu_avgpool", "bn_train_act", "softmax_nll"};
		std::stringstream res;
		for (const fused_group& grp : plan_fusion(nodes, training != 0))
		{
			res << kKinds[grp.kind] << " " << (grp.entry_point.empty() ? "-" : grp.entry_point) << " members=";
			for (size_t k = 0; k < grp.members.size(); ++k)
				res << (k ? "," : "") << nodes[grp.members[k]].name;
			res << " residual=" << (grp.residual_input.empty() ? "-" : grp.residual_input) << " elided=";
			if (grp.elided.empty())
				res << "-";
			for (size_t k = 0; k < grp.elided.size(); ++k)
				res << (k ? "," : "") << nodes[grp.elided[k]].name;
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
		g_fusion_error = e.what();
		return -1;
	}
}
