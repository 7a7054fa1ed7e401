// SPDX-License-Identifier: Apache-2.0
// Source compatibility: programs written against the original include layout find the same
// declarations here.
#pragma once
#include "cs/modules.h"
