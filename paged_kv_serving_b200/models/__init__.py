"""Architectures. Importing this package registers every built-in architecture."""

from paged_kv_serving_b200.models.layout import LayerCall, ModelLayout, collect_param_specs
from paged_kv_serving_b200.models.llama_toy_decoder import LlamaToyDecoder
from paged_kv_serving_b200.models.revupel import Revupel
from paged_kv_serving_b200.models.rodelix import Rodelix
from paged_kv_serving_b200.models.segetar import Segetar
from paged_kv_serving_b200.models.tiburax import Tiburax

__all__ = ["LayerCall", "LlamaToyDecoder", "ModelLayout", "Revupel", "Rodelix", "Segetar", "Tiburax", "collect_param_specs"]
