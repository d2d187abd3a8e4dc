"""Expert parallelism: runtime, engines and the ElasticBuffer API (the only parallel dimension of this library)."""
