/* placeholder translation unit; the HNSW baseline is added in hnsw_baseline.c */
int orc_hnsw_present(void) { return 0; }
