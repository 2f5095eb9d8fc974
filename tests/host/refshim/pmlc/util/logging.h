// Stand-in for the reference's pmlc/util/logging.h (easylogging++ behind it): its tests include it, the ones
// compiled here log nothing through it.
#pragma once
#include <iostream>
#define IVLOG(level, message) \
  do {                        \
  } while (0)
