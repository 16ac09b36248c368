from .store_backend import IdStore, create_process_group_from_store

__all__ = ["IdStore", "create_process_group_from_store"]
