// Stand-in for the TensorFlow header of the same name (test infrastructure only).
#include "tf_stub.h"
