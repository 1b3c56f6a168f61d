// Empty stand-in: the plain-backend headers include <boost/uuid/uuid.hpp> but the hot-path
// translation units never name a uuid. Test infrastructure only.
#pragma once
namespace boost { namespace uuids { struct uuid { unsigned char data[16]; }; } }
