"""B200-native (sm_100a) kernels for one decoder layer's decode step, behind the per-op entry
points of Kushagrabainsla/muse-spark-open: proj, attention, moe, layer (prepare / kernel_fn)."""
