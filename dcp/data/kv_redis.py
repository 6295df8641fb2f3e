from dcp_b200.data.kv_store import KVStore as RedisKVStore, KVServer as RedisServer  # noqa: F401
