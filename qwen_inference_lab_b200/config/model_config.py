"""Typed model configuration, read from a checkpoint's own ``config.json`` keys.

Keys, defaults and rejections follow the reference's ``ModelConfig``
(qil/config.py:8-45): eight required positive integers, ``rms_norm_eps``,
``rope_theta``, ``attention_bias``, ``tie_word_embeddings`` and ``eos_token_id``
with the same defaults; ``model_type`` other than ``qwen3``, a ``rope_scaling``,
``use_sliding_window``, a ``layer_types`` entry other than ``full_attention`` and a
``hidden_act`` other than ``silu`` are refused.  No size lives in code: every part
of the model is built from these fields alone.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
import json
import math
from pathlib import Path


class ConfigError(ValueError):
    """A config.json that this engine cannot run."""


_REQUIRED_INTS = (
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
)


@dataclass(frozen=True)
class Qwen3Config:
    """Dense Qwen3 decoder (reference: qil/config.py:8-22)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    attention_bias: bool = False
    tie_word_embeddings: bool = True
    eos_token_id: int | list | None = None

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    def __post_init__(self):
        for name in _REQUIRED_INTS:
            value = getattr(self, name)
            if type(value) is not int or value < 1:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for half-split rotation, got {self.head_dim}")
        for name in ("rms_norm_eps", "rope_theta"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, (int, float)) \
                    or not math.isfinite(value) or value <= 0:
                raise ConfigError(f"{name} must be positive and finite, got {value!r}")
        for name in ("attention_bias", "tie_word_embeddings"):
            if type(getattr(self, name)) is not bool:
                raise ConfigError(f"{name} must be a boolean")
        eos = self.eos_token_id
        if eos is not None:
            items = eos if isinstance(eos, list) else [eos]
            if any(type(t) is not int or t < 0 for t in items):
                raise ConfigError("eos_token_id must be an integer, a list of integers or null")

    @property
    def eos_token_ids(self) -> frozenset:
        eos = self.eos_token_id
        if eos is None:
            return frozenset()
        return frozenset(eos if isinstance(eos, list) else [eos])

    @classmethod
    def from_dict(cls, data: dict) -> "Qwen3Config":
        """Validate a parsed config.json (reference: qil/config.py:34-45)."""
        if data.get("model_type", cls.model_type) != cls.model_type:
            raise ConfigError(
                f"model_type {data.get('model_type')!r} is not the dense '{cls.model_type}' decoder")
        if data.get("rope_scaling") is not None:
            raise ConfigError("rope_scaling is not supported: only unscaled rotary positions")
        if data.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window is not supported: every layer attends to all keys")
        if any(kind != "full_attention" for kind in data.get("layer_types") or []):
            raise ConfigError("layer_types must all be 'full_attention'")
        if data.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {data.get('hidden_act')!r} is not supported: only 'silu'")
        missing = [name for name in _REQUIRED_INTS if name not in data]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        known = {f.name for f in fields(cls)}
        return cls(**{key: data[key] for key in known if key in data})

    def to_dict(self) -> dict:
        data = {f.name: getattr(self, f.name) for f in fields(self)}
        data["architectures"] = [self.architecture]
        data["model_type"] = self.model_type
        data["hidden_act"] = "silu"
        return data


def read_config_json(directory) -> dict:
    path = Path(directory) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {directory}")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data


_MIXER_KEYS = {
    "attention": {"heads", "kv_heads", "dim", "vdim"},         # "scale" defaults to dim^-1/2
    "gla": {"heads", "dim", "vdim", "tau"},
}


class VirulixConfig:
    """Virulix: a decoder whose layers are listed one by one in config.json.

    ``vocab``, ``width``, ``norm.eps`` and ``layers``: each layer names its mixer (``type``: ``attention`` or
    ``gla``), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: ``dense``, ``moe``
    or null).  The configuration is kept as the dictionary it came in; this class checks it and answers
    the few questions the engine asks.  The design has no position table, so ``max_positions`` (not a key
    of the design; 2**20 unless given) only bounds what a request may ask for: the cache is the limit.
    """
    architecture = "Virulix"
    model_type = "virulix"

    def __init__(self, data: dict):
        self.data = data
        for key in ("vocab", "width"):
            if type(data.get(key)) is not int or data[key] < 1:
                raise ConfigError(f"{key} must be a positive integer, got {data.get(key)!r}")
        eps = (data.get("norm") or {}).get("eps")
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not eps > 0:
            raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for index, layer in enumerate(layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in _MIXER_KEYS:
                raise ConfigError(f"layers[{index}].type {kind!r} is not one of {sorted(_MIXER_KEYS)}")
            if not isinstance(mixer, dict) or _MIXER_KEYS[kind] - set(mixer):
                raise ConfigError(f"layers[{index}].mixer lacks {sorted(_MIXER_KEYS[kind] - set(mixer or {}))}")
            if kind == "attention":
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"layers[{index}]: {mixer['heads']} heads do not divide into {mixer['kv_heads']} kv heads")
                source = mixer.get("kv_from")
                if source is not None:
                    if type(source) is not int or not 0 <= source < index or layers[source].get("type") != "attention" \
                            or layers[source]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"layers[{index}].mixer.kv_from must name an earlier attention layer with "
                                          f"keys and values of its own")
                    theirs = layers[source]["mixer"]
                    if any(theirs[k] != mixer[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"layers[{index}] and layers[{source}] differ in the shape of keys and values")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    if type(mlp.get("ff")) is not int or mlp["ff"] < 1:
                        raise ConfigError(f"layers[{index}].mlp.ff must be a positive integer")
                elif mlp.get("kind") == "moe":
                    router, expert = mlp.get("router") or {}, mlp.get("expert") or {}
                    if not {"experts", "top"} <= set(router) or not {"ff", "limit"} <= set(expert):
                        raise ConfigError(f"layers[{index}].mlp needs router.experts, router.top, expert.ff and expert.limit")
                    if not 1 <= router["top"] <= router["experts"]:
                        raise ConfigError(f"layers[{index}].mlp: {router['top']} of {router['experts']} experts")
                    shared = mlp.get("shared")
                    if shared is not None and not {"ff", "limit"} <= set(shared):
                        raise ConfigError(f"layers[{index}].mlp.shared needs ff and limit")
                else:
                    raise ConfigError(f"layers[{index}].mlp.kind {mlp.get('kind')!r} is neither dense nor moe")
        self.vocab_size, self.width, self.eps = data["vocab"], data["width"], float(eps)
        self.layers = layers
        self.max_positions = int(data.get("max_positions", 1 << 20))
        eos = data.get("eos_token_id")
        self.eos_token_ids = frozenset() if eos is None else frozenset(eos if isinstance(eos, list) else [eos])

    @classmethod
    def from_dict(cls, data: dict) -> "VirulixConfig":
        if data.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {cls.architecture}")
        return cls(json.loads(json.dumps(data)))

    def to_dict(self) -> dict:
        return json.loads(json.dumps(self.data)) | {"architecture": self.architecture}

    def __eq__(self, other):
        return isinstance(other, VirulixConfig) and self.to_dict() == other.to_dict()


def _positive_int(value) -> bool:
    return type(value) is int and value >= 1


class DebisunConfig:
    """Debisun: a decoder whose layers are listed one by one in config.json.

    ``vocab``, ``width``, ``norm.eps``, ``token_side.dim`` (the size of a layer's slice of the per-token side
    table; absent: no side input) and ``layers``: every layer is an ``attention`` mixer with its sizes and
    constants (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv`` taps, ``softcap``, ``bias_max``,
    ``mask.size``) and a feed-forward (``mlp``: ``dense`` with ``ff``; ``moe`` with ``router`` (``experts``,
    ``top``, ``identity``, ``scale``), ``expert.ff`` and optionally ``shared.ff``; or null).  The configuration is
    kept as the dictionary it came in; this class checks it and answers the few questions the engine asks.
    The number of rows of a layer's distance table is a size that only the tensor gives.  The design has no
    position table: ``max_positions`` (not a key of the design; 2**20 unless given) only bounds a request.
    """
    architecture = "Debisun"
    model_type = "debisun"

    def __init__(self, data: dict):
        self.data = data
        for key in ("vocab", "width"):
            if not _positive_int(data.get(key)):
                raise ConfigError(f"{key} must be a positive integer, got {data.get(key)!r}")
        eps = (data.get("norm") or {}).get("eps")
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not eps > 0:
            raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
        side = data.get("token_side")
        if side is not None and not _positive_int((side or {}).get("dim")):
            raise ConfigError(f"token_side.dim must be a positive integer, got {side!r}")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for index, layer in enumerate(layers):
            where = f"layers[{index}]"
            if layer.get("type") != "attention":
                raise ConfigError(f"{where}.type {layer.get('type')!r} is not 'attention'")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                if not _positive_int(mixer.get(key)):
                    raise ConfigError(f"{where}.mixer.{key} must be a positive integer, got {mixer.get(key)!r}")
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"{where}: {mixer['heads']} heads do not divide into {mixer['kv_heads']} kv heads")
            for key in ("scale", "softcap"):
                value = mixer.get(key)
                if key == "softcap" and value is None:
                    continue
                if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
                    raise ConfigError(f"{where}.mixer.{key} must be a positive number, got {value!r}")
            taps = mixer.get("conv")
            if taps is not None and not _positive_int(taps):
                raise ConfigError(f"{where}.mixer.conv must be a positive number of taps, got {taps!r}")
            if not _positive_int(mixer.get("bias_max")):
                raise ConfigError(f"{where}.mixer.bias_max must be a positive integer, got {mixer.get('bias_max')!r}")
            mask = mixer.get("mask")
            if mask is not None and not _positive_int((mask or {}).get("size")):
                raise ConfigError(f"{where}.mixer.mask.size must be a positive integer, got {mask!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                if not _positive_int(mlp.get("ff")):
                    raise ConfigError(f"{where}.mlp.ff must be a positive integer")
            elif mlp.get("kind") == "moe":
                router, expert = mlp.get("router") or {}, mlp.get("expert") or {}
                if not _positive_int(router.get("experts")) or not _positive_int(router.get("top")) \
                        or not _positive_int(expert.get("ff")):
                    raise ConfigError(f"{where}.mlp needs router.experts, router.top and expert.ff")
                identity = router.get("identity", 0)
                if type(identity) is not int or identity < 0:
                    raise ConfigError(f"{where}.mlp.router.identity must be a non-negative integer")
                if router["top"] > router["experts"] + identity:
                    raise ConfigError(f"{where}.mlp: {router['top']} of {router['experts']} + {identity} router outputs")
                scale = router.get("scale", 1.0)
                if isinstance(scale, bool) or not isinstance(scale, (int, float)):
                    raise ConfigError(f"{where}.mlp.router.scale must be a number")
                shared = mlp.get("shared")
                if shared is not None and not _positive_int(shared.get("ff")):
                    raise ConfigError(f"{where}.mlp.shared.ff must be a positive integer")
            else:
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is neither dense nor moe")
        self.vocab_size, self.width, self.eps = data["vocab"], data["width"], float(eps)
        self.side_dim = side["dim"] if side else 0
        self.layers = layers
        self.max_positions = int(data.get("max_positions", 1 << 20))
        eos = data.get("eos_token_id")
        self.eos_token_ids = frozenset() if eos is None else frozenset(eos if isinstance(eos, list) else [eos])

    @classmethod
    def from_dict(cls, data: dict) -> "DebisunConfig":
        if data.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {cls.architecture}")
        return cls(json.loads(json.dumps(data)))

    def to_dict(self) -> dict:
        return json.loads(json.dumps(self.data)) | {"architecture": self.architecture}

    def __eq__(self, other):
        return isinstance(other, DebisunConfig) and self.to_dict() == other.to_dict()


def _positive_number(value) -> bool:
    return not isinstance(value, bool) and isinstance(value, (int, float)) and value > 0


class LarolornConfig:
    """Larolorn: a decoder whose layers are listed one by one in config.json, some of them running with another
    layer's weights.

    ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (what a normed branch is multiplied by on its way into the
    stream), ``logit_scale`` and ``layers``.  A layer is a ``latent_attention`` mixer (``heads``, ``dim``,
    ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot`` with ``base`` and ``dims``, ``mask.size`` the window) or a
    ``parallel`` one: ``left`` a grouped attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot``,
    ``mask.size`` the chunk) beside ``right`` a linear attention with a fixed decay per head (``heads``, ``dim``,
    ``vdim``, ``decay``); and a feed-forward (``mlp``: ``dense`` with ``ff`` and ``limit``, or null).
    ``weights_of: j`` names the layer whose tensors the layer runs with (cache and state stay its own).
    The configuration is kept as the dictionary it came in; this class checks it and answers the few questions
    the engine asks.  ``max_positions`` (not a key of the design; 2**20 unless given) only bounds a request.
    """
    architecture = "Larolorn"
    model_type = "larolorn"

    def __init__(self, data: dict):
        self.data = data
        for key in ("vocab", "width"):
            if not _positive_int(data.get(key)):
                raise ConfigError(f"{key} must be a positive integer, got {data.get(key)!r}")
        eps = (data.get("norm") or {}).get("eps")
        if not _positive_number(eps):
            raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
        for key in ("residual_mult", "logit_scale"):
            value = data.get(key, 1.0)
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise ConfigError(f"{key} must be a number, got {value!r}")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for index, layer in enumerate(layers):
            where = f"layers[{index}]"
            kind, mixer = layer.get("type"), layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind == "latent_attention":
                self._check_sizes(where, mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
                self._check_rotation(where, mixer, mixer["rot_dim"])
                if mixer["rot"]["dims"] != mixer["rot_dim"]:
                    raise ConfigError(f"{where}: the rotated part has {mixer['rot_dim']} dimensions, rot.dims says {mixer['rot']['dims']}")
                self._check_mask(where, mixer)
            elif kind == "parallel":
                left, right = mixer.get("left"), mixer.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise ConfigError(f"{where}.mixer needs a left and a right mixer")
                self._check_sizes(where + ".left", left, ("heads", "kv_heads", "dim", "vdim"))
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}: {left['heads']} heads do not divide into {left['kv_heads']} kv heads")
                self._check_rotation(where + ".left", left, left["dim"])
                self._check_mask(where + ".left", left)
                self._check_sizes(where + ".right", right, ("heads", "dim", "vdim"))
                decay = right.get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"] \
                        or any(isinstance(v, bool) or not isinstance(v, (int, float)) or not 0 <= v <= 1 for v in decay):
                    raise ConfigError(f"{where}.right.decay must give one decay in [0, 1] per head")
            else:
                raise ConfigError(f"{where}.type {kind!r} is neither latent_attention nor parallel")
            for m in ([mixer] if kind == "latent_attention" else [mixer["left"]]):
                if not _positive_number(m.get("scale")):
                    raise ConfigError(f"{where}: scale must be a positive number, got {m.get('scale')!r}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not dense")
                if not _positive_int(mlp.get("ff")) or not _positive_number(mlp.get("limit")):
                    raise ConfigError(f"{where}.mlp needs a positive ff and limit")
            source = layer.get("weights_of")
            if source is not None:
                if type(source) is not int or not 0 <= source < len(layers) or source == index \
                        or layers[source].get("weights_of") is not None:
                    raise ConfigError(f"{where}.weights_of must name another layer that has tensors of its own")
                theirs = layers[source]
                if any(theirs.get(k) != layer.get(k) for k in ("type", "mixer", "mlp")):
                    raise ConfigError(f"{where} and layers[{source}] share weights but differ in type, mixer or mlp")
        self.vocab_size, self.width, self.eps = data["vocab"], data["width"], float(eps)
        self.residual_mult, self.logit_scale = float(data.get("residual_mult", 1.0)), float(data.get("logit_scale", 1.0))
        self.layers = layers
        self.max_positions = int(data.get("max_positions", 1 << 20))
        eos = data.get("eos_token_id")
        self.eos_token_ids = frozenset() if eos is None else frozenset(eos if isinstance(eos, list) else [eos])

    @staticmethod
    def _check_sizes(where, mixer, keys):
        for key in keys:
            if not _positive_int(mixer.get(key)):
                raise ConfigError(f"{where}.{key} must be a positive integer, got {mixer.get(key)!r}")

    @staticmethod
    def _check_rotation(where, mixer, most):
        rot = mixer.get("rot")
        if not isinstance(rot, dict) or not _positive_number(rot.get("base")) or not _positive_int(rot.get("dims")) \
                or rot["dims"] % 2 or rot["dims"] > most:
            raise ConfigError(f"{where}.rot needs a positive base and an even number of dims, at most {most}; got {rot!r}")

    @staticmethod
    def _check_mask(where, mixer):
        if not _positive_int((mixer.get("mask") or {}).get("size")):
            raise ConfigError(f"{where}.mask.size must be a positive integer, got {mixer.get('mask')!r}")

    @classmethod
    def from_dict(cls, data: dict) -> "LarolornConfig":
        if data.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {cls.architecture}")
        return cls(json.loads(json.dumps(data)))

    def to_dict(self) -> dict:
        return json.loads(json.dumps(self.data)) | {"architecture": self.architecture}

    def __eq__(self, other):
        return isinstance(other, LarolornConfig) and self.to_dict() == other.to_dict()


class GogotarConfig:
    """Gogotar: a decoder whose layers are listed one by one in config.json, a run of them looped.

    ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (what a token's row is multiplied by), ``logit_softcap``
    (logits <- cap * tanh(logits / cap)), ``layers`` and ``loop`` (``start``, ``stop``, ``times``: layers
    start .. stop - 1 run ``times`` times in a row with the same tensors, every pass with a cache of its own).
    A layer is an ``attention`` mixer (``heads``, ``kv_heads``, ``dim``, ``vdim`` = ``dim`` since the values are the
    keys, ``scale``, ``softcap``, ``rot`` with ``base``, ``dims`` and optionally ``scaling`` with ``factor``, ``low``,
    ``high``, ``original``; ``mask.size`` the chunk) or a ``latent_attention`` one (``heads``, ``dim``, ``vdim``,
    ``kv_rank``, ``q_rank``, ``scale``), and a feed-forward: ``mlp`` null, ``dense`` (``ff``, ``limit``) or ``moe``
    (``expert.ff``, ``router.experts``, ``router.top``).  The configuration is kept as the dictionary it came in;
    this class checks it and answers the few questions the engine asks.  ``max_positions`` (not a key of the design;
    2**20 unless given) only bounds a request.
    """
    architecture = "Gogotar"
    model_type = "gogotar"

    def __init__(self, data: dict):
        self.data = data
        for key in ("vocab", "width"):
            if not _positive_int(data.get(key)):
                raise ConfigError(f"{key} must be a positive integer, got {data.get(key)!r}")
        eps = (data.get("norm") or {}).get("eps")
        if not _positive_number(eps):
            raise ConfigError(f"norm.eps must be a positive number, got {eps!r}")
        scale = (data.get("embedding") or {}).get("scale", 1.0)
        if not _positive_number(scale):
            raise ConfigError(f"embedding.scale must be a positive number, got {scale!r}")
        cap = data.get("logit_softcap")
        if cap is not None and not _positive_number(cap):
            raise ConfigError(f"logit_softcap must be a positive number or absent, got {cap!r}")
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for index, layer in enumerate(layers):
            where = f"layers[{index}]"
            kind, mixer = layer.get("type"), layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind == "attention":
                LarolornConfig._check_sizes(where, mixer, ("heads", "kv_heads", "dim"))
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}: {mixer['heads']} heads do not divide into {mixer['kv_heads']} kv heads")
                if mixer.get("vdim", mixer["dim"]) != mixer["dim"]:
                    raise ConfigError(f"{where}: the values are the keys, so vdim must be dim ({mixer['dim']})")
                LarolornConfig._check_rotation(where, mixer, mixer["dim"])
                scaling = mixer["rot"].get("scaling")
                if scaling is not None and (not all(_positive_number(scaling.get(k)) for k in ("factor", "low", "high", "original"))
                                            or scaling["low"] >= scaling["high"]):
                    raise ConfigError(f"{where}.rot.scaling needs positive factor, low < high and original; got {scaling!r}")
                if mixer.get("mask") is not None:
                    LarolornConfig._check_mask(where, mixer)
                if mixer.get("softcap") is not None and not _positive_number(mixer["softcap"]):
                    raise ConfigError(f"{where}.softcap must be a positive number or absent")
            elif kind == "latent_attention":
                LarolornConfig._check_sizes(where, mixer, ("heads", "dim", "vdim", "kv_rank", "q_rank"))
            else:
                raise ConfigError(f"{where}.type {kind!r} is neither attention nor latent_attention")
            if not _positive_number(mixer.get("scale")):
                raise ConfigError(f"{where}: scale must be a positive number, got {mixer.get('scale')!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                if not _positive_int(mlp.get("ff")) or not _positive_number(mlp.get("limit")):
                    raise ConfigError(f"{where}.mlp needs a positive ff and limit")
            elif mlp.get("kind") == "moe":
                router, expert = mlp.get("router") or {}, mlp.get("expert") or {}
                if not _positive_int(expert.get("ff")) or not _positive_int(router.get("experts")) \
                        or not _positive_int(router.get("top")) or router["top"] > router["experts"]:
                    raise ConfigError(f"{where}.mlp needs expert.ff, router.experts and router.top <= experts")
            else:
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is neither dense nor moe")
        loop = data.get("loop")
        if loop is not None:
            if not all(type(loop.get(k)) is int for k in ("start", "stop", "times")) \
                    or not 0 <= loop["start"] <= loop["stop"] <= len(layers) or loop["times"] < 1:
                raise ConfigError(f"loop needs 0 <= start <= stop <= {len(layers)} and times >= 1, got {loop!r}")
        self.vocab_size, self.width, self.eps = data["vocab"], data["width"], float(eps)
        self.embedding_scale, self.logit_softcap = float(scale), float(cap or 0.0)
        self.layers = layers
        self.max_positions = int(data.get("max_positions", 1 << 20))
        eos = data.get("eos_token_id")
        self.eos_token_ids = frozenset() if eos is None else frozenset(eos if isinstance(eos, list) else [eos])

    def layer_runs(self) -> list:
        """The layers' indices in the order they run."""
        count, loop = len(self.layers), self.data.get("loop")
        if loop is None:
            return list(range(count))
        return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] \
            + list(range(loop["stop"], count))

    @classmethod
    def from_dict(cls, data: dict) -> "GogotarConfig":
        if data.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"architecture {data.get('architecture')!r} is not {cls.architecture}")
        return cls(json.loads(json.dumps(data)))

    def to_dict(self) -> dict:
        return json.loads(json.dumps(self.data)) | {"architecture": self.architecture}

    def __eq__(self, other):
        return isinstance(other, GogotarConfig) and self.to_dict() == other.to_dict()
