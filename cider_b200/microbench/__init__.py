"""Stand-alone CUDA micro-benchmarks that calibrate the rooflines quoted for the
kernels: what the hardware does with the instruction or the copy alone.

    python -m cider_b200.microbench            # build (nvcc, sm_100a) and run both
    python -m cider_b200.microbench mma_rate   # tcgen05.mma issue / completion rate by shape
    python -m cider_b200.microbench hbm_stream # 26 MB read once per launch: plain loads vs bulk-copy rings

The binaries are written next to the sources (git-ignored)."""
