// Minimal stand-in for boost::format, enough for the error-message formatting the
// nnForge plain-backend sources perform ("%1%"-style positional arguments, operator%, str()).
// Test infrastructure only: it lets the reference's own CPU sources compile where Boost is absent.
#pragma once
#include <sstream>
#include <string>
#include <vector>

namespace boost
{
	class format
	{
	public:
		explicit format(const std::string& pattern) : pattern_(pattern) {}

		template <class T>
		format& operator%(const T& value)
		{
			std::ostringstream s;
			s << value;
			args_.push_back(s.str());
			return *this;
		}

		std::string str() const
		{
			std::string out;
			for (size_t i = 0; i < pattern_.size(); ++i)
			{
				if (pattern_[i] == '%')
				{
					size_t j = i + 1;
					size_t index = 0;
					while (j < pattern_.size() && pattern_[j] >= '0' && pattern_[j] <= '9')
						index = index * 10 + static_cast<size_t>(pattern_[j++] - '0');
					if (j < pattern_.size() && pattern_[j] == '%' && j > i + 1)
					{
						if (index >= 1 && index <= args_.size())
							out += args_[index - 1];
						i = j;
						continue;
					}
				}
				out += pattern_[i];
			}
			return out;
		}

	private:
		std::string pattern_;
		std::vector<std::string> args_;
	};

	inline std::ostream& operator<<(std::ostream& os, const format& f) { return os << f.str(); }
}
