// Force-included when the reference's host-only encoder source is compiled with g++ instead of
// nvcc: nvcc's headers leak an unqualified `max` that the source relies on at one place.
#include <algorithm>
#include <unordered_set>
using std::max;
