// TEST INFRASTRUCTURE ONLY: see dnnl.hpp in this directory.
#pragma once
#include "../../dnnl.hpp"
