from .dist import StatelessGroup, stateless_init_process_group

__all__ = ["StatelessGroup", "stateless_init_process_group"]
