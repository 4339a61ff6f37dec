from .builder import BaseMaskBuilder, MaskBuilderFactory, SectionedMaskBuilder
from .pipeline import Pipeline, filter_by_length

__all__ = ["BaseMaskBuilder", "MaskBuilderFactory", "SectionedMaskBuilder", "Pipeline", "filter_by_length"]
