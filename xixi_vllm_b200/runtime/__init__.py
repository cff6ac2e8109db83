"""Per-rank compute runtime: worker lifecycle, model runner, batch staging, KV pool, graphs."""
