// Include-case shim: the reference's src/Utils.cpp:1 includes "micrograd/utils.h"
// while the header on disk is include/micrograd/Utils.h; on a case-sensitive
// file system the reference only compiles with this forwarding header on the path.
#pragma once
#include "micrograd/Utils.h"
