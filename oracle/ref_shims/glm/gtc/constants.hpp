// Stand-in for glm/gtc/constants.hpp: only pi<T>() is used by the reference sources.
#pragma once
#include "../glm.hpp"
namespace glm {
template <typename T> GLM_FUNC_QUALIFIER constexpr T pi() { return T(3.14159265358979323846264338327950288L); }
}  // namespace glm
