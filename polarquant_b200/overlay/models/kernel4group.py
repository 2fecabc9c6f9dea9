"""Overlay for the reference's ``models.kernel4group``: put the ``overlay`` directory ahead of
the reference checkout on ``sys.path`` and ``from models.kernel4group import ...`` resolves here."""
from polarquant_b200.kernel4group import attention_decode_forward_triton_impl  # noqa: F401
