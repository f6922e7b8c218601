"""``vllm.general_plugins`` entry point of the B200 attention backend.

Counterpart of the reference's plugin module (python/pth_flash_attn/plugin.py:28-46): vLLM
calls :func:`register` in every process it starts, before an attention backend is chosen,
and the function only records a class path under the one enum member reserved for
out-of-tree backends (``AttentionBackendEnum.CUSTOM``).  Nothing else is imported here, so
a server that never selects ``--attention-backend CUSTOM`` loads neither the CUDA library
nor the backend module.

An entry-point declaration for a packaging file::

    [project.entry-points."vllm.general_plugins"]
    pth_flash_attn_b200 = "pth_flash_attn_b200.plugin:register"
"""
from __future__ import annotations

import logging

BACKEND_CLASS_PATH = "pth_flash_attn_b200.vllm_backend.PthFlashAttnBackend"

_log = logging.getLogger(__name__)


def register() -> bool:
    """Claim ``CUSTOM`` for this backend unless another plugin holds it.

    Returns True if the member now points at this backend.  A different class that is
    already registered there is left alone (with a warning): replacing it would silently
    change what ``--attention-backend CUSTOM`` means for that installation.
    """
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    member = AttentionBackendEnum.CUSTOM
    taken = member.is_overridden()
    if taken and member.get_path() != BACKEND_CLASS_PATH:
        _log.warning("pth_flash_attn_b200: AttentionBackendEnum.CUSTOM already names %s; not replacing it",
                     member.get_path())
        return False
    if not taken:
        register_backend(member, BACKEND_CLASS_PATH)
    return True
