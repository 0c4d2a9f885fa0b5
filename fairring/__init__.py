"""Drop-in name of the library: ``import fairring`` registers the "fairring"
backend exactly as the reference package does (fairring/__init__.py:49), so

    import fairring
    torch.distributed.init_process_group("fairring")

keeps working unchanged.  Everything lives in :mod:`fairring_b200`.
"""

from fairring_b200 import (  # noqa: F401
    __version__,
    create_process_group_fairring,
    get_backend,
    launch_count,
    options_from_env,
)
