// Empty stand-in: lets the reference headers be parsed without the cusp library, which only
// the reference's Matrix-Market loaders (not compiled here) use.
#pragma once
