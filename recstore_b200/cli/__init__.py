"""Command-line drivers mirroring the reference's executables (perf_emb, test_emb, perf_rec_model, KG training, DLRM)."""
