"""Helpers that behave sensibly with and without an initialised process group."""
import torch.distributed as dist


class DistUtil:
    """World-size / rank queries that fall back to a single process."""
    @staticmethod
    def _is_dist_avail_and_initialized():
        return dist.is_available() and dist.is_initialized()

    @classmethod
    def get_world_size(cls, group=None):
        return dist.get_world_size(group) if cls._is_dist_avail_and_initialized() else 1

    @classmethod
    def get_rank(cls, group=None):
        return dist.get_rank(group) if cls._is_dist_avail_and_initialized() else 0

    @classmethod
    def is_main_process(cls):
        return cls.get_rank() == 0

    @classmethod
    def backend(cls, group=None):
        return dist.get_backend(group) if cls._is_dist_avail_and_initialized() else None

    @staticmethod
    def broadcast_object_list(object_list, src=0, group=None, device=None):
        """Broadcast picklable objects; a no-op without a process group."""
        if DistUtil._is_dist_avail_and_initialized():
            dist.broadcast_object_list(object_list, src=src, group=group, device=device)
        return object_list
