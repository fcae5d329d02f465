"""B200-native (sm_100a) implementation of microxcaling's quantization path."""
