"""Historical import location of the dtype-code tables (see comfy_kitchen.ops)."""
from comfy_kitchen.ops import DTYPE_CODE_TO_DTYPE, DTYPE_TO_CODE  # noqa: F401
