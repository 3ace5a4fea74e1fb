// Stand-in header: the reference includes this file but uses nothing from it
// beyond what mlx/array.h already declares.
#pragma once
#include "mlx/array.h"
