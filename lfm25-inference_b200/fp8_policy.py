"""Loader of the reference's FP8 precision policy file.

The reference selects which linear sites run in E4M3, and with which static scales, from a JSON document
(`Fp8PrecisionPolicy`, src/model/quantization.rs:44-68; its promoted policy is
docs/benchmarks/fp8/selected-policy.json): `schema_version`, `name`, `source`, `decode_only` and a list of sites
`{site, enabled, activation_strategy, weight_strategy, activation_scale, weight_scale, local_nrmse, local_cosine,
expected_decode_saving_us}` where a scale is `{clip_amax, quantize_multiplier, dequantize_multiplier}`
(`ScalarScale`, :159-173: q = 448 / c, d = c / 448).  Site names are `layers.<i>.mlp.gate_up`,
`layers.<i>.mlp.down`, `lm_head` and the attention / convolution projections.  A file in that schema loads unchanged.
"""
from __future__ import annotations

import json
import math
import re
from dataclasses import dataclass


@dataclass(frozen=True)
class ScalarScale:
    clip_amax: float
    quantize_multiplier: float
    dequantize_multiplier: float

    @classmethod
    def from_json(cls, node: dict, what: str) -> "ScalarScale":
        try:
            scale = cls(float(node["clip_amax"]), float(node["quantize_multiplier"]),
                        float(node["dequantize_multiplier"]))
        except (KeyError, TypeError, ValueError) as error:
            raise ValueError(f"{what}: malformed scale ({error})") from error
        for value in (scale.clip_amax, scale.quantize_multiplier, scale.dequantize_multiplier):
            if not (math.isfinite(value) and value > 0.0):
                raise ValueError(f"{what}: scale values must be finite and positive")
        return scale


@dataclass(frozen=True)
class Fp8SitePolicy:
    site: str
    enabled: bool
    activation_scale: ScalarScale
    weight_scale: ScalarScale
    activation_strategy: str = "amax"
    weight_strategy: str = "amax"


@dataclass(frozen=True)
class Fp8PrecisionPolicy:
    name: str
    source: str
    decode_only: bool
    sites: tuple

    def enabled_sites(self) -> list[str]:
        return [site.site for site in self.sites if site.enabled]

    def site(self, name: str) -> Fp8SitePolicy | None:
        for site in self.sites:
            if site.site == name:
                return site
        return None

    def layers_with(self, kind: str) -> tuple:
        """Layer indices whose `layers.<i>.mlp.<kind>` site is enabled (kind: gate_up | down)."""
        pattern = re.compile(rf"^layers\.(\d+)\.mlp\.{re.escape(kind)}$")
        found = []
        for site in self.sites:
            match = pattern.match(site.site)
            if match and site.enabled:
                found.append(int(match.group(1)))
        return tuple(sorted(found))

    def lm_head_enabled(self) -> bool:
        site = self.site("lm_head")
        return site is not None and site.enabled


def parse_fp8_policy(document: dict) -> Fp8PrecisionPolicy:
    if not isinstance(document, dict) or "sites" not in document:
        raise ValueError("FP8 policy: missing `sites`")
    if int(document.get("schema_version", 0)) != 1:
        raise ValueError(f"FP8 policy: unsupported schema_version {document.get('schema_version')!r}")
    sites, seen = [], set()
    for index, node in enumerate(document["sites"]):
        name = node.get("site") if isinstance(node, dict) else None
        if not isinstance(name, str) or not name:
            raise ValueError(f"FP8 policy: site {index} has no name")
        if name in seen:
            raise ValueError(f"FP8 policy: site {name!r} appears twice")
        seen.add(name)
        if not isinstance(node.get("enabled"), bool):
            raise ValueError(f"FP8 policy: site {name!r} has no boolean `enabled`")
        sites.append(Fp8SitePolicy(
            name, node["enabled"], ScalarScale.from_json(node.get("activation_scale"), f"{name}.activation_scale"),
            ScalarScale.from_json(node.get("weight_scale"), f"{name}.weight_scale"),
            str(node.get("activation_strategy", "amax")), str(node.get("weight_strategy", "amax"))))
    return Fp8PrecisionPolicy(str(document.get("name", "")), str(document.get("source", "")),
                              bool(document.get("decode_only", True)), tuple(sites))


def load_fp8_policy(path: str) -> Fp8PrecisionPolicy:
    with open(path) as handle:
        return parse_fp8_policy(json.load(handle))
