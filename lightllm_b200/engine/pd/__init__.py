from .kv_transport import KVReceiver, KVSender, PageHeader  # noqa: F401
