"""Multi-GPU runtime: peer memory, fused data-parallel step, meshes."""
