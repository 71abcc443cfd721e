// TEST INFRASTRUCTURE ONLY.  Stand-in for the build-generated DistConv
// configuration header: every optional backend is off (CPU "Ref" backend only).
#pragma once
#include "h2_config.hpp"
