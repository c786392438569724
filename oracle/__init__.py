"""CPU oracle of the packed ragged step. TEST INFRASTRUCTURE ONLY: the shipped package never imports it."""
