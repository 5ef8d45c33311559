// See core.h of this directory: the stand-in formats through operator<< already.
#pragma once
#include "core.h"
