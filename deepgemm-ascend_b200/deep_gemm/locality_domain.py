"""Locality-domain helpers kept as no-ops for import compatibility (deep_gemm/locality_domain.py:1-26):
B200 exposes one uniform memory domain per GPU."""


def get_num_locality_domains() -> int:
    return 1


def is_localization_available() -> bool:
    return False


def localize(tensor, *args, **kwargs):
    return tensor


def is_localized(tensor) -> bool:
    return False


def destroy_localizer() -> None:
    return None
