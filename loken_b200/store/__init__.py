"""Model stores: where model files live on disk and how a name resolves to them."""
