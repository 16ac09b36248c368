from .naive_router import NaiveRouter, RouterClient, launch_router

__all__ = ["NaiveRouter", "RouterClient", "launch_router"]
