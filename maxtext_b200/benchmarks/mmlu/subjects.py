"""The 57 MMLU subjects with the field and the broad area each belongs to (the grouping published with the benchmark,
Hendrycks et al. 2021), kept as one table: `subject field`, fields grouped into areas below."""
from __future__ import annotations

_TABLE = """
abstract_algebra math | anatomy health | astronomy physics | business_ethics business | clinical_knowledge health
college_biology biology | college_chemistry chemistry | college_computer_science computer_science | college_mathematics math
college_medicine health | college_physics physics | computer_security computer_science | conceptual_physics physics
econometrics economics | electrical_engineering engineering | elementary_mathematics math | formal_logic philosophy
global_facts other | high_school_biology biology | high_school_chemistry chemistry | high_school_computer_science computer_science
high_school_european_history history | high_school_geography geography | high_school_government_and_politics politics
high_school_macroeconomics economics | high_school_mathematics math | high_school_microeconomics economics
high_school_physics physics | high_school_psychology psychology | high_school_statistics math | high_school_us_history history
high_school_world_history history | human_aging health | human_sexuality culture | international_law law | jurisprudence law
logical_fallacies philosophy | machine_learning computer_science | management business | marketing business
medical_genetics health | miscellaneous other | moral_disputes philosophy | moral_scenarios philosophy | nutrition health
philosophy philosophy | prehistory history | professional_accounting other | professional_law law | professional_medicine health
professional_psychology psychology | public_relations politics | security_studies politics | sociology culture
us_foreign_policy politics | virology health | world_religions philosophy
"""

FIELD_OF = {s: f.replace("_", " ") for s, f in (item.split() for line in _TABLE.strip().splitlines() for item in line.split(" | "))}

AREAS = {
    "STEM": ("physics", "chemistry", "biology", "computer science", "math", "engineering"),
    "humanities": ("history", "philosophy", "law"),
    "social sciences": ("politics", "culture", "economics", "geography", "psychology"),
    "other (business, health, misc.)": ("other", "business", "health"),
}
AREA_OF = {f: a for a, fs in AREAS.items() for f in fs}
assert len(FIELD_OF) == 57 and all(f in AREA_OF for f in FIELD_OF.values())
