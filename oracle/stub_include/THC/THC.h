// Stand-in for the PyTorch-0.3 THC umbrella header, which no longer exists.  The reference's
// kernel files include it but use nothing from it except printf.
#include <cstdio>
