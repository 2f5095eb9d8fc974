// Stand-in: the reference's test sources include gmock for matchers their fixture uses; the fixture
// here (plaidml/testenv.h of this directory) compares by itself.
#pragma once
#include "gtest/gtest.h"
