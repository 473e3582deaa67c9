"""B200-native deformable kernels: same package layout and public names as the
reference project's ``deformable_kernels`` package, backed by libdk_b200.so."""
