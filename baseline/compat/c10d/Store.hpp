// Old include path of PyTorch 1.11; see ProcessGroup.hpp in this directory.
#pragma once
#include <c10d/ProcessGroup.hpp>
