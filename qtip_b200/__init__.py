"""qtip_b200: B200-native (sm_100a) kernels for the QTIP quantized-linear path."""
