"""Task layer: ``.family`` / ``.task`` documents, the goal-predicate language and its device tape, placement sampling,
reward shaping, a family environment and the family training drivers (reference: noeira/tasks/)."""
from .predicates import BoundGoal, GoalState, Term, bind_goal, evaluate, evaluate_cuda, family_tables, parse_goal, require_evaluable
from .sampler import InitTable, Placements, sample_placements
from .shaping import ShapedGoalReward
from .spec import (FamilySpec, InitSpec, JointInitSpec, RegionSpec, SlotSpec, TaskSpec, load_family, load_task, order_inits,
                   parse_family, parse_init, parse_region, parse_slot, parse_task, validate_task_against_family)
